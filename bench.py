#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Llama 3.2 1B with random weights:
decode at batch 8 with 1,024 tokens of context per request (the headline
``value``, decoded tokens per second), the same through the Python entry point
with host tokens in and out (``e2e``), decode at batch 1 and 64 (``points``),
one 2,048-token prefill (``prefill``) and the decode step's memory roofline
(``roofline``).  One JSON line is printed.  A step is one decode step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_3_2_1B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
    head_dim=64, num_hidden_layers=16, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=131072, torch_dtype="bfloat16")
CONTEXT = 1024            # tokens each decoding request holds
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)     # used only if MEASURED_PEAKS.json is absent


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            data = json.load(open(path))
            return dict(hbm_gbs=float(data["hbm_gbs"]), bf16_tflops=float(data["bf16_tflops"]),
                        bf16_tflops_sustained=float(data.get("bf16_tflops_sustained", data["bf16_tflops"]))), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timing runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.proc = [], None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons}


def model_folder(cfg_dict, seed=0):
    """The model folder with random weights (written once per machine into the temporary folder)."""
    from railgun_b200.config.registry import architecture_name, architecture_of
    from railgun_b200.weights.random_init import write_random_model
    if "hidden_size" in cfg_dict:
        tag = f"rg_bench_L{cfg_dict['num_hidden_layers']}_H{cfg_dict['hidden_size']}_V{cfg_dict['vocab_size']}_s{seed}"
    else:
        import hashlib
        tag = f"rg_bench_{hashlib.sha1(json.dumps(cfg_dict, sort_keys=True).encode()).hexdigest()[:12]}_s{seed}"
    d = os.path.join(tempfile.gettempdir(), tag)
    if not (os.path.exists(os.path.join(d, "model.safetensors")) and os.path.exists(os.path.join(d, "config.json"))):
        tmp = d + f".tmp{os.getpid()}"
        config = architecture_of(architecture_name(cfg_dict)).config_from_dict(cfg_dict)
        write_random_model(config, seed, tmp)
        if os.path.exists(d):
            import shutil
            shutil.rmtree(d, ignore_errors=True)
        os.replace(tmp, d)
    return d


def decode_bytes(cfg, batch, context, kv_bytes_per_token):
    """Bytes a decode step has to read: every weight once, and the cache of the live requests."""
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * d * H + nh * d * H + 3 * I * H + 2 * H
    weights = (L * per_layer + V * H + H) * 2              # the head's matrix once, tied or not
    embedding_rows = batch * H * 2                          # of the embedding table only the tokens' rows
    return weights + embedding_rows + batch * context * kv_bytes_per_token


def prefill_flops(cfg, T):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * T * L * ((nh + 2 * nkv) * d * H + nh * d * H + 3 * I * H)
    attn = L * nh * 2 * 2 * d * (T * (T + 1) // 2)          # causal: QK^T and PV
    return linear + attn + 2 * V * H


def decode_tools(runner, V, rng):
    """``fill_contexts``, ``DecodeLoop`` and ``time_decode`` over one runner: the decode steps that generation
    launches, timed in windows with CUDA events."""
    import numpy as np
    import torch
    from railgun_b200.engine.batch import StepEntry
    from railgun_b200 import ops
    launches = ops.launch_counter()

    def fill_contexts(batch, first_id, context=CONTEXT):
        """Prefill ``batch`` requests of ``context`` tokens each; returns their ids and first sampled tokens."""
        ids = list(range(first_id, first_id + batch))
        toks = []
        for rid in ids:
            prompt = rng.integers(0, V, size=context).tolist()
            lg = runner.step([StepEntry(rid, prompt, [context - 1])])
            toks.append(int(ops.argmax(lg).item()))
        return np.asarray(ids, dtype=np.int64), np.asarray(toks, dtype=np.int32)

    class DecodeLoop:
        """Decode steps for requests in the cache, launched as generation launches them (``Engine.step``): the
        first from host tokens, every later one while the one before it runs, its token ids staying on the
        device; but no step's tokens are read here.  ``log`` [n, rows] receives every step's tokens."""

        def __init__(self, ids, toks, log=None):
            self.ids, self.log, self.done, self.follow = ids, log, 0, None
            runner.decode_step_flat(ids, toks)
            self._note(runner.last_greedy)

        def _note(self, sampled):
            if self.log is not None:
                self.log[self.done, :len(self.ids)].copy_(sampled[:len(self.ids)])
            self.done += 1

        def run(self, n):
            for _ in range(n):
                nxt = runner.decode_follow(self.ids, self.follow)
                if nxt is None:
                    raise RuntimeError("the cache has no room for the timed decode steps")
                if self.follow is not None:
                    runner.alloc.advance(self.ids, 1)      # the step before is committed once its successor is packed
                self.follow = nxt
                self._note(nxt.static.sampled)

        def close(self):
            if self.follow is not None:
                runner.alloc.advance(self.ids, 1)
            torch.cuda.synchronize()

    def time_decode(batch, steps, warmup, first_id, context=CONTEXT, min_seconds=0.3):
        """Windows of exactly ``steps`` decode steps each, timed with CUDA events, until ``min_seconds`` are
        covered (three windows at least); before each window the requests go back to ``context`` tokens, so every
        window reads the same amount of cache.  Returns the median window."""
        ids, toks = fill_contexts(batch, first_id, context)
        back = np.full(batch, context, dtype=np.int32)
        windows, n_launch, total = [], 0, 0.0
        while len(windows) < 3 or (total < min_seconds and len(windows) < 200):
            runner.alloc.commit_many(ids, back)
            loop = DecodeLoop(ids, toks)
            loop.run(warmup - 1)
            torch.cuda.synchronize()
            n0 = launches.value
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            loop.run(steps)
            t1.record()
            torch.cuda.synchronize()
            loop.close()
            n_launch = launches.value - n0
            ms = t0.elapsed_time(t1)
            windows.append(ms / steps)
            total += ms * 1e-3
        runner.check_device_errors()
        runner.end(ids.tolist())
        ms = sorted(windows)[len(windows) // 2]
        return batch / ms * 1e3, ms, n_launch, len(windows)

    return fill_contexts, DecodeLoop, time_decode


def run_ours(args):
    import numpy as np
    import torch
    from railgun_b200.engine.batch import StepEntry
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    from railgun_b200 import ops

    cfg = dict(LLAMA_3_2_1B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk, pk_src = peaks()
    mdir = model_folder(cfg)
    page = 16
    pool_tokens = 64 * 8192                                # the cache pool: 64 sequences x 8,192 tokens
    eng = Engine(mdir, dtype="bfloat16", block_size=page, num_gpu_blocks=pool_tokens // page, max_num_seqs=64,
                 max_num_batched_tokens=8192, max_model_len=8192)
    runner = eng.runner
    V = cfg["vocab_size"]
    rng = np.random.default_rng(0)
    kv_per_token = runner.cache.bytes_per_token()
    launches = ops.launch_counter()

    fill_contexts, DecodeLoop, time_decode = decode_tools(runner, V, rng)

    def hbm_frac(batch, ms, steps, warmup, context=CONTEXT):
        bytes_step = decode_bytes(cfg, batch, context + warmup + steps // 2, kv_per_token)
        achieved = bytes_step / (ms * 1e-3) / 1e9
        return achieved, achieved / pk["hbm_gbs"]

    def e2e_window(prompts, steps, warmup):
        """``steps`` calls of Engine.step with every request decoding: host tokens in, host tokens out."""
        rids = [eng.add_request(p, SamplingParams(max_new_tokens=steps + warmup + 2)) for p in prompts]
        tokens = {r: [] for r in rids}
        while True:                                        # until all prompts are in the cache
            out = eng.step()
            for r, t in out or ():
                tokens[r].append(t)
            if out is not None and len(out) == len(prompts):
                break
        for _ in range(warmup):
            for r, t in eng.step():
                tokens[r].append(t)
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for _ in range(steps):
            for r, t in eng.step():
                tokens[r].append(t)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - w0
        h2d = eng.runner.last_h2d_bytes
        for r in rids:
            eng.abort(r)
            eng.collect(r)
        return seconds * 1e3 / steps, h2d, [tokens[r] for r in rids]

    def check_tokens(prompts, n=24):
        """The timed loop against the entry point: the same prompts through Engine.step, token by token on the
        host, and through ``DecodeLoop`` after the same prefill; every token of every step must be equal."""
        _, _, by_engine = e2e_window(prompts, n - 1, 1)
        rids = [eng.add_request(p, SamplingParams(max_new_tokens=n + 2)) for p in prompts]
        while True:
            out = eng.step()
            if out is not None and len(out) == len(prompts):
                break
        first = dict(out)
        ids = np.asarray(rids, dtype=np.int64)
        log = torch.zeros((n, len(rids)), dtype=torch.int32, device=runner.device)
        loop = DecodeLoop(ids, np.asarray([first[r] for r in rids], dtype=np.int32), log)
        loop.run(n - 1)
        loop.close()
        by_loop = log.cpu().numpy()
        for r in rids:
            eng.abort(r)
            eng.collect(r)
        return all([first[r]] + by_loop[:, i].tolist() == by_engine[i][:n + 1] for i, r in enumerate(rids))

    if args.mode == "decode":                              # a short run of one decode batch (for profiling)
        tok_s, ms_step, n_launch, _ = time_decode(args.batch, args.steps, args.warmup, 1000, args.context,
                                                  min_seconds=0.0 if args.windows == 1 else 0.3)
        print(json.dumps({"mode": "decode", "batch": args.batch, "context": args.context, "tok_s": round(tok_s, 1),
                          "hbm_frac": round(hbm_frac(args.batch, ms_step, args.steps, args.warmup, args.context)[1], 4),
                          "ms_per_step": round(ms_step, 4), "gpu_launches": n_launch,
                          "layers": cfg["num_hidden_layers"]}))
        return 0
    if args.mode == "prefill":
        prompt = rng.integers(0, V, size=args.tokens).tolist()
        times = []
        for i in range(args.warmup + args.steps):
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            runner.step([StepEntry(7000 + i, prompt, [args.tokens - 1])])
            t1.record()
            torch.cuda.synchronize()
            runner.end([7000 + i])
            times.append(t0.elapsed_time(t1))
        ms = sorted(times[args.warmup:])[len(times[args.warmup:]) // 2]
        print(json.dumps({"mode": "prefill", "tokens": args.tokens, "ms": round(ms, 3),
                          "tok_s": round(args.tokens / ms * 1e3, 1), "layers": cfg["num_hidden_layers"],
                          "frac": round(prefill_flops(cfg, args.tokens) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0

    prompts = [rng.integers(0, V, size=CONTEXT).tolist() for _ in range(8)]
    checked = bool(check_tokens(prompts))
    with ClockSampler() as clocks:
        tok_s, ms_step, n_launch, n_windows = time_decode(8, args.steps, args.warmup, 1000)
    clock_summary = clocks.summary()
    points = {}
    for b in (1, 64):
        b_tok_s, b_ms, _, _ = time_decode(b, args.steps, args.warmup, 2000 + 100 * b)
        points[f"decode_b{b}"] = round(b_tok_s, 1)
        points[f"decode_b{b}_ms_per_step"] = round(b_ms, 4)
        points[f"decode_b{b}_frac"] = round(hbm_frac(b, b_ms, args.steps, args.warmup)[1], 4)

    # prefill of 2,048 tokens, logits at the last position
    prompt = rng.integers(0, V, size=PREFILL_TOKENS).tolist()
    pf_ms = []
    for i in range(args.warmup + 9):
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        runner.step([StepEntry(5000 + i, prompt, [PREFILL_TOKENS - 1])])
        t1.record()
        torch.cuda.synchronize()
        runner.end([5000 + i])
        if i >= args.warmup:
            pf_ms.append(t0.elapsed_time(t1))
    runner.check_device_errors()
    pf = sorted(pf_ms)[len(pf_ms) // 2]
    flops = prefill_flops(cfg, PREFILL_TOKENS)

    # end to end through the entry point: host tokens in, host tokens out, every step; the median window
    e2e, seconds = [], 0.0
    while len(e2e) < 3 or (seconds < 0.3 and len(e2e) < 200):
        ms, h2d, _ = e2e_window(prompts, args.steps, args.warmup)
        e2e.append(ms)
        seconds += ms * args.steps * 1e-3
    e2e_ms = sorted(e2e)[len(e2e) // 2]
    d2h = 8 * 4

    achieved, frac = hbm_frac(8, ms_step, args.steps, args.warmup)
    line = {
        "metric": "decode tok/s at batch 8 (Llama 3.2 1B sizes, 1,024-token contexts)",
        "value": round(tok_s, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
        "impl": "ours", "checked": checked,
        "config": {
            "model": "Llama-3.2-1B sizes, random weights", "layers": cfg["num_hidden_layers"],
            "layers_of_named_config": full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": 8,
            "seq_len": CONTEXT, "block_size": page, "kv_pool_tokens": pool_tokens, "parallelism": "none (1 GPU)",
            "l2": "inputs larger than L2 (2.5 GB of weights per step)", "peaks": pk_src,
            "timing": f"median of {n_windows} windows of {args.steps} steps",
        },
        "e2e": {"value": round(8 / e2e_ms * 1e3, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "frac": round(hbm_frac(8, e2e_ms, args.steps, args.warmup)[1], 4), "windows": len(e2e)},
        "gpu_launches": int(n_launch),
        "prefill": {"value": round(PREFILL_TOKENS / pf * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pf, 3),
                    "frac": round(flops / (pf * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(frac, 4)},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


def dizatar_sizes(name):
    """(Dizatar configuration, the Llama configuration of equal width, layer runs and vocabulary beside it)."""
    def diz(width, heads, dim, rot, vdim, rank, experts, identity, top, ff, shared, vocab):
        layer = dict(type="latent_attention",
                     mixer=dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, scale=(dim + rot) ** -0.5,
                                rot=dict(base=10000.0, dims=rot)),
                     mlp=dict(kind="moe", router=dict(experts=experts, identity=identity, top=top), expert=dict(ff=ff),
                              shared=dict(ff=shared)))
        return dict(architecture="Dizatar", width=width, vocab=vocab, norm=dict(eps=1e-6), residual_mult=0.6,
                    logit_softcap=30.0, loop=dict(start=1, stop=3, times=2), layers=[layer] * 4)

    def llama(width, heads, kv, ff, vocab, runs):
        return dict(architectures=["LlamaForCausalLM"], hidden_size=width, num_attention_heads=heads,
                    num_key_value_heads=kv, head_dim=64, num_hidden_layers=runs, intermediate_size=ff, vocab_size=vocab,
                    rope_theta=500000.0, rope_scaling=None, tie_word_embeddings=True, rms_norm_eps=1e-5,
                    max_position_embeddings=131072, torch_dtype="bfloat16")

    if name == "w2048":      # 16 heads of 128 + 64 over a latent of 512; 32 experts of 1,024, 4 of 34 chosen
        return diz(2048, 16, 128, 64, 128, 512, 32, 2, 4, 1024, 2048, 32768), llama(2048, 32, 8, 8192, 32768, 6)
    if name == "w1024":      # 8 heads of 64 + 32 over a latent of 256; 16 experts of 512, 2 of 17 chosen
        return diz(1024, 8, 64, 32, 64, 256, 16, 1, 2, 512, 1024, 32768), llama(1024, 16, 4, 4096, 32768, 6)
    raise ValueError(name)


def dizatar_runs(cfg):
    """The layers in the order they run (a looped span ``times`` times)."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return list(range(n)), 0
    order = list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))
    return order, loop["times"]


def dizatar_decode_bytes(cfg, batch, context):
    """Bytes a decode step of ``batch`` tokens has to read: attention and shared-expert weights once per layer run,
    the experts that the batch is expected to touch under uniform routing, the head, and the latent cache."""
    W, V = cfg["width"], cfg["vocab"]
    order, passes = dizatar_runs(cfg)
    total = V * W * 2 + passes * 2 * W * W * 2
    for i in order:
        m, f = cfg["layers"][i]["mixer"], cfg["layers"][i]["mlp"]
        H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        total += (H * (dn + dr) * W + (R + dr) * W + H * dn * R + H * dv * R + W * H * dv) * 2
        total += batch * context * (R + dr) * 2
        if f:
            E, ident, top, F = f["router"]["experts"], f["router"]["identity"], f["router"]["top"], f["expert"]["ff"]
            touched = E * (1.0 - (1.0 - top / (E + ident)) ** batch)
            total += touched * 3 * F * W * 2 + (E + ident) * W * 4
            if f.get("shared"):
                total += 3 * f["shared"]["ff"] * W * 2
    return total


def dizatar_prefill_flops(cfg, T):
    """FLOPs of one prompt of T tokens as the engine computes it: attention in the expanded form where the
    engine expands prompts (keys of dn + dr and values of dv numbers per head, plus the expansion of every
    context token through U_k and U_v), else in the absorbed form (scores over latent + rotated numbers, values
    over the latent)."""
    W, V = cfg["width"], cfg["vocab"]
    order, passes = dizatar_runs(cfg)
    total = 2 * V * W + passes * 2 * T * 2 * W * W
    for i in order:
        m, f = cfg["layers"][i]["mixer"], cfg["layers"][i]["mlp"]
        H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        total += 2 * T * (H * (dn + dr) * W + (R + dr) * W + H * dn * R + H * dv * R + W * H * dv)
        d = dn + dr
        if d % 16 == 0 and d <= 256 and dv <= d and d + dv < 2 * R + dr:
            total += H * 2 * (d + dv) * (T * (T + 1) // 2) + 2 * T * R * H * (dn + dv)
        else:
            total += H * 2 * (2 * R + dr) * (T * (T + 1) // 2)
        if f:
            E, ident, top, F = f["router"]["experts"], f["router"]["identity"], f["router"]["top"], f["expert"]["ff"]
            total += 2 * T * (top * E / (E + ident) * 3 * F * W + (E + ident) * W)
            if f.get("shared"):
                total += 2 * T * 3 * f["shared"]["ff"] * W
    return total


def run_dizatar(args):
    """Prefill and decode throughput of Dizatar at layer sizes of real models (random weights), beside the dense
    GQA Llama of equal width, number of layer runs and vocabulary.  One JSON line per model and size."""
    import numpy as np
    import torch
    from railgun_b200.engine.batch import StepEntry
    from railgun_b200.engine.engine import Engine
    page, pool_tokens = 16, 64 * 4096
    pk, pk_src = peaks()
    for size in (args.sizes.split(",") if args.sizes else ["w1024", "w2048"]):
        for label, cfg in zip(("dizatar", "llama"), dizatar_sizes(size)):
            mdir = model_folder(cfg)
            eng = Engine(mdir, dtype="bfloat16", block_size=page, num_gpu_blocks=pool_tokens // page, max_num_seqs=64,
                         max_num_batched_tokens=8192, max_model_len=4096)
            runner = eng.runner
            V = cfg.get("vocab", cfg.get("vocab_size"))
            rng = np.random.default_rng(0)
            _, _, time_decode = decode_tools(runner, V, rng)
            line = {"mode": "dizatar", "size": size, "model": label, "layer_runs": len(runner.model.order),
                    "cache_bytes_per_token": runner.cache.bytes_per_token()}
            for b in (8, 64):
                tok_s, ms, n_launch, _ = time_decode(b, args.steps, args.warmup, 1000 * b, args.context)
                line[f"decode_b{b}_tok_s"], line[f"decode_b{b}_ms"] = round(tok_s, 1), round(ms, 4)
                line[f"decode_b{b}_launches_per_step"] = n_launch // args.steps
                ctx = args.context + args.warmup + args.steps // 2
                by = (dizatar_decode_bytes(cfg, b, ctx) if label == "dizatar"
                      else decode_bytes(cfg, b, ctx, runner.cache.bytes_per_token()))
                line[f"decode_b{b}_GB_per_step"] = round(by / 1e9, 3)
                line[f"decode_b{b}_frac_hbm"] = round(by / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)
            prompt = rng.integers(0, V, size=args.tokens).tolist()
            times = []
            for i in range(args.warmup + 7):
                torch.cuda.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                runner.step([StepEntry(7000 + i, prompt, [args.tokens - 1])])
                t1.record()
                torch.cuda.synchronize()
                runner.end([7000 + i])
                times.append(t0.elapsed_time(t1))
            runner.check_device_errors()
            ms = sorted(times[args.warmup:])[len(times[args.warmup:]) // 2]
            fl = dizatar_prefill_flops(cfg, args.tokens) if label == "dizatar" else prefill_flops(cfg, args.tokens)
            line.update(prefill_tokens=args.tokens, prefill_ms=round(ms, 3), prefill_tok_s=round(args.tokens / ms * 1e3, 1),
                        prefill_TFLOP=round(fl / 1e12, 3), prefill_frac_flops=round(fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3),
                        peaks=pk_src)
            print(json.dumps(line), flush=True)
            del eng, runner, time_decode
            torch.cuda.empty_cache()
    return 0


def rupulix_sizes(name):
    """(Rupulix configuration, the Llama configuration of equal width, layer runs and vocabulary beside it)."""
    def rup(width, heads, kv, d, lat_heads, dim, rot, rank, window, blocks, ff, vocab):
        par = dict(type="parallel", mlp=dict(kind="dense", ff=ff), mixer=dict(
            left=dict(heads=heads, kv_heads=kv, dim=d, vdim=d, rot=dict(base=10000.0, dims=d // 2), scale=d ** -0.5),
            right=dict(width=width, blocks=blocks, conv=4), left_scale=0.5, right_scale=0.5))
        lat = dict(type="latent_attention", mlp=dict(kind="dense", ff=ff), mixer=dict(
            heads=lat_heads, dim=dim, rot_dim=rot, vdim=dim, kv_rank=rank, scale=(dim + rot) ** -0.5,
            rot=dict(base=10000.0, dims=rot), mask=dict(size=window)))
        return dict(architecture="Rupulix", width=width, vocab=vocab, norm=dict(eps=1e-6), streams=2, logit_scale=1.0,
                    loop=dict(start=1, stop=3, times=2), layers=[par, lat, par, lat])

    def llama(width, heads, kv, ff, vocab, runs):
        return dict(architectures=["LlamaForCausalLM"], hidden_size=width, num_attention_heads=heads,
                    num_key_value_heads=kv, head_dim=64, num_hidden_layers=runs, intermediate_size=ff, vocab_size=vocab,
                    rope_theta=500000.0, rope_scaling=None, tie_word_embeddings=True, rms_norm_eps=1e-5,
                    max_position_embeddings=131072, torch_dtype="bfloat16")

    if name == "w2048":      # 16 heads of 128 on 2 key/value heads beside a recurrence of 2,048 in 8 blocks; 16 heads of 128 + 64 over a latent of 512, window 512
        return rup(2048, 16, 2, 128, 16, 128, 64, 512, 512, 8, 8192, 32768), llama(2048, 32, 8, 8192, 32768, 6)
    if name == "w1024":      # 8 heads of 64 on 2 key/value heads beside a recurrence of 1,024 in 4 blocks; 8 heads of 64 + 32 over a latent of 256, window 512
        return rup(1024, 8, 2, 64, 8, 64, 32, 256, 512, 4, 4096, 32768), llama(1024, 16, 4, 4096, 32768, 6)
    raise ValueError(name)


def rupulix_decode_bytes(cfg, batch, context):
    """Bytes a decode step has to read: every weight of every layer run, the head, and what the live requests keep
    (a windowed layer's cache only as far back as its window)."""
    W, V = cfg["width"], cfg["vocab"]
    order, _ = dizatar_runs(cfg)
    total = V * W * 2
    for i in order:
        L = cfg["layers"][i]
        m = L["mixer"]
        if L["type"] == "latent_attention":
            H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            total += (H * (dn + dr) * W + (R + dr) * W + H * dn * R + H * dv * R + W * H * dv) * 2
            total += batch * min(context, (m.get("mask") or {}).get("size", context)) * (R + dr) * 2
        else:
            a, r = m["left"], m["right"]
            H, G, d, dv, C, B = a["heads"], a["kv_heads"], a["dim"], a["vdim"], r["width"], r["blocks"]
            total += ((H + G) * d * W + G * dv * W + W * H * dv + 3 * C * W) * 2 + 2 * C * (C // B) * 4
            total += batch * (context * G * (d + dv) * 2 + r["conv"] * C * 4)
        if L["mlp"]:
            total += 2 * L["mlp"]["ff"] * W * 2
    return total


def rupulix_prefill_flops(cfg, T):
    """FLOPs of one prompt of T tokens by the design's own arithmetic: products, attention over the keys a query
    sees (the latent layers in the absorbed form the engine runs), the heads' score mixing, the gates."""
    W, V = cfg["width"], cfg["vocab"]
    order, _ = dizatar_runs(cfg)
    total = 2 * V * W
    for i in order:
        L = cfg["layers"][i]
        m = L["mixer"]
        if L["type"] == "latent_attention":
            H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            win = (m.get("mask") or {}).get("size", T)
            pairs = sum(min(t + 1, win) for t in range(T))
            total += 2 * T * (H * (dn + dr) * W + (R + dr) * W + H * dn * R + H * dv * R + W * H * dv)
            total += H * 2 * (2 * R + dr) * pairs
        else:
            a, r = m["left"], m["right"]
            H, G, d, dv, C, B = a["heads"], a["kv_heads"], a["dim"], a["vdim"], r["width"], r["blocks"]
            total += 2 * T * ((H + G) * d * W + G * dv * W + W * H * dv + 3 * C * W + 2 * C * (C // B))
            total += (H * 2 * (d + dv) + 2 * H * H) * (T * (T + 1) // 2)
        if L["mlp"]:
            total += 2 * T * 2 * L["mlp"]["ff"] * W
    return total


def run_rupulix(args):
    """Prefill and decode throughput of Rupulix at layer sizes of real models (random weights), beside the dense
    GQA Llama of equal width, number of layer runs and vocabulary.  One JSON line per model and size."""
    import numpy as np
    import torch
    from railgun_b200.engine.batch import StepEntry
    from railgun_b200.engine.engine import Engine
    page, pool_tokens = 16, 64 * 4096
    pk, pk_src = peaks()
    for size in (args.sizes.split(",") if args.sizes else ["w1024", "w2048"]):
        for label, cfg in zip(("rupulix", "llama"), rupulix_sizes(size)):
            mdir = model_folder(cfg)
            eng = Engine(mdir, dtype="bfloat16", block_size=page, num_gpu_blocks=pool_tokens // page, max_num_seqs=64,
                         max_num_batched_tokens=8192, max_model_len=4096)
            runner = eng.runner
            V = cfg.get("vocab", cfg.get("vocab_size"))
            rng = np.random.default_rng(0)
            _, _, time_decode = decode_tools(runner, V, rng)
            line = {"mode": "rupulix", "size": size, "model": label, "layer_runs": len(runner.model.order),
                    "cache_bytes_per_token": runner.cache.bytes_per_token()}
            for b in (8, 64):
                tok_s, ms, n_launch, _ = time_decode(b, args.steps, args.warmup, 1000 * b, args.context)
                line[f"decode_b{b}_tok_s"], line[f"decode_b{b}_ms"] = round(tok_s, 1), round(ms, 4)
                line[f"decode_b{b}_launches_per_step"] = n_launch // args.steps
                ctx = args.context + args.warmup + args.steps // 2
                by = (rupulix_decode_bytes(cfg, b, ctx) if label == "rupulix"
                      else decode_bytes(cfg, b, ctx, runner.cache.bytes_per_token()))
                line[f"decode_b{b}_GB_per_step"] = round(by / 1e9, 3)
                line[f"decode_b{b}_frac_hbm"] = round(by / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)
            prompt = rng.integers(0, V, size=args.tokens).tolist()
            times = []
            for i in range(args.warmup + 7):
                torch.cuda.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                runner.step([StepEntry(7000 + i, prompt, [args.tokens - 1])])
                t1.record()
                torch.cuda.synchronize()
                runner.end([7000 + i])
                times.append(t0.elapsed_time(t1))
            runner.check_device_errors()
            ms = sorted(times[args.warmup:])[len(times[args.warmup:]) // 2]
            fl = rupulix_prefill_flops(cfg, args.tokens) if label == "rupulix" else prefill_flops(cfg, args.tokens)
            line.update(prefill_tokens=args.tokens, prefill_ms=round(ms, 3), prefill_tok_s=round(args.tokens / ms * 1e3, 1),
                        prefill_TFLOP=round(fl / 1e12, 3), prefill_frac_flops=round(fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3),
                        peaks=pk_src)
            print(json.dumps(line), flush=True)
            del eng, runner, time_decode
            torch.cuda.empty_cache()
    return 0


def mepatar_sizes(name):
    """(Mepatar configuration, the Rupulix configuration of equal width, layer runs and vocabulary beside it)."""
    def mep(width, heads, kv, d, window, ff, experts, top, eff, vocab):
        ret = dict(type="retention", mixer=dict(heads=heads, dim=d, vdim=d, rot=dict(base=10000.0, dims=d),
                                                decay=[1.0 - 2.0 ** (-5 - 0.4 * i) for i in range(heads)]))
        dlt = dict(type="delta", mixer=dict(heads=heads, kv_heads=heads // 2, dim=d, vdim=d, conv=4))
        att = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv, dim=d, vdim=d, scale=d ** -0.5,
                                                rot=dict(base=10000.0, dims=d // 2), mask=dict(size=window, keep_first=4)))
        dense = dict(kind="dense", ff=ff)
        moe = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=eff, limit=7.0))
        layers = [dict(ret, mlp=dense), dict(dlt, mlp=moe), dict(att, mlp=moe), dict(ret, mlp=moe), dict(dlt, mlp=dense),
                  dict(att, mlp=dense)]
        return dict(architecture="Mepatar", width=width, vocab=vocab, norm=dict(eps=1e-6, groups=4),
                    embedding=dict(scale=width ** 0.5), canon=dict(taps=4), layers=layers)

    if name == "w2048":      # 16 heads of 128 (2 key/value heads, window 512 keeping 4); 32 experts of 2,048, 4 chosen
        return mep(2048, 16, 2, 128, 512, 8192, 32, 4, 2048, 32768), rupulix_sizes(name)[0]
    if name == "w1024":      # 8 heads of 128 (2 key/value heads, window 512 keeping 4); 16 experts of 1,024, 4 chosen
        return mep(1024, 8, 2, 128, 512, 4096, 16, 4, 1024, 32768), rupulix_sizes(name)[0]
    raise ValueError(name)


def mepatar_decode_bytes(cfg, batch, context):
    """Bytes a decode step has to read or write: the weights of every layer (of the experts, those that `batch`
    tokens can reach at most), the head, and what the live requests keep: matrix states in 32-bit (read and
    written), convolution tails, and an attention layer's cache as far back as its window and kept tokens."""
    W, V = cfg["width"], cfg["vocab"]
    K0 = (cfg.get("canon") or {}).get("taps", 0)
    total = V * W * 2
    for L in cfg["layers"]:
        m = L["mixer"]
        if K0:
            total += batch * (K0 - 1) * W * 4 * 2
        if L["type"] == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            total += (2 * H * d + 2 * H * dv) * W * 2 + W * H * dv * 2 + batch * H * d * dv * 4 * 2
        elif L["type"] == "delta":
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            total += (2 * G * d + 2 * H * dv + 2 * H) * W * 2 + W * H * dv * 2
            total += batch * (H * d * dv * 4 * 2 + (K - 1) * (2 * G * d + H * dv) * 4 * 2)
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mask = m.get("mask") or {}
            seen = min(context, mask["size"] + mask.get("keep_first", 0)) if mask.get("size") else context
            total += ((H + G) * d + G * dv) * W * 2 + W * H * dv * 2 + batch * seen * G * 2 * max(d, dv) * 2
        f = L["mlp"]
        if f and f["kind"] == "dense":
            total += 3 * f["ff"] * W * 2
        elif f:
            r, e = f["router"], f["expert"]
            total += r["experts"] * W * 2 + min(r["experts"], batch * r["top"]) * 3 * e["ff"] * W * 2
    return total


def mepatar_prefill_flops(cfg, T):
    """FLOPs of one prompt of T tokens by the design's own arithmetic: products, the chosen experts, attention
    over the keys a query sees, and the matrix states' updates and read-outs (4 d dv per head and token)."""
    W, V = cfg["width"], cfg["vocab"]
    total = 2 * V * W
    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            total += 2 * T * ((2 * H * d + 2 * H * dv) * W + W * H * dv) + T * H * 4 * d * dv
        elif L["type"] == "delta":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            total += 2 * T * ((2 * G * d + 2 * H * dv + 2 * H) * W + W * H * dv) + T * H * 6 * d * dv
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mask = m.get("mask") or {}
            win, keep = mask.get("size", 0), mask.get("keep_first", 0)
            pairs = sum(min(t + 1, win + min(keep, max(0, t + 1 - win))) if win else t + 1 for t in range(T))
            total += 2 * T * (((H + G) * d + G * dv) * W + W * H * dv) + H * 2 * (d + dv) * pairs
        f = L["mlp"]
        if f and f["kind"] == "dense":
            total += 2 * T * 3 * f["ff"] * W
        elif f:
            total += 2 * T * (f["router"]["experts"] * W + f["router"]["top"] * 3 * f["expert"]["ff"] * W)
    return total


def run_mepatar(args):
    """Prefill and decode throughput of Mepatar at layer sizes of real models (random weights), beside Rupulix
    (the framework's other design with state slots, a window and parallel branches) at equal width, number of
    layer runs and vocabulary.  One JSON line per model and size."""
    import numpy as np
    import torch
    from railgun_b200.engine.batch import StepEntry
    from railgun_b200.engine.engine import Engine
    page, pool_tokens = 16, 64 * 4096
    pk, pk_src = peaks()
    for size in (args.sizes.split(",") if args.sizes else ["w1024", "w2048"]):
        for label, cfg in zip(("mepatar", "rupulix"), mepatar_sizes(size)):
            mdir = model_folder(cfg)
            eng = Engine(mdir, dtype="bfloat16", block_size=page, num_gpu_blocks=pool_tokens // page, max_num_seqs=64,
                         max_num_batched_tokens=8192, max_model_len=4096)
            runner = eng.runner
            V = cfg["vocab"]
            rng = np.random.default_rng(0)
            _, _, time_decode = decode_tools(runner, V, rng)
            line = {"mode": "mepatar", "size": size, "model": label, "layer_runs": len(runner.model.order),
                    "cache_bytes_per_token": runner.cache.bytes_per_token()}
            for b in (8, 64):
                tok_s, ms, n_launch, _ = time_decode(b, args.steps, args.warmup, 1000 * b, args.context)
                line[f"decode_b{b}_tok_s"], line[f"decode_b{b}_ms"] = round(tok_s, 1), round(ms, 4)
                line[f"decode_b{b}_launches_per_step"] = n_launch // args.steps
                ctx = args.context + args.warmup + args.steps // 2
                by = mepatar_decode_bytes(cfg, b, ctx) if label == "mepatar" else rupulix_decode_bytes(cfg, b, ctx)
                line[f"decode_b{b}_GB_per_step"] = round(by / 1e9, 3)
                line[f"decode_b{b}_frac_hbm"] = round(by / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)
            prompt = rng.integers(0, V, size=args.tokens).tolist()
            times = []
            for i in range(args.warmup + 7):
                torch.cuda.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                runner.step([StepEntry(7000 + i, prompt, [args.tokens - 1])])
                t1.record()
                torch.cuda.synchronize()
                runner.end([7000 + i])
                times.append(t0.elapsed_time(t1))
            runner.check_device_errors()
            ms = sorted(times[args.warmup:])[len(times[args.warmup:]) // 2]
            fl = mepatar_prefill_flops(cfg, args.tokens) if label == "mepatar" else rupulix_prefill_flops(cfg, args.tokens)
            line.update(prefill_tokens=args.tokens, prefill_ms=round(ms, 3), prefill_tok_s=round(args.tokens / ms * 1e3, 1),
                        prefill_TFLOP=round(fl / 1e12, 3), prefill_frac_flops=round(fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3),
                        peaks=pk_src)
            print(json.dumps(line), flush=True)
            del eng, runner, time_decode
            torch.cuda.empty_cache()
    return 0


def kasarax_sizes(name):
    """(Kasarax configuration, the Mepatar configuration of equal width, layers and vocabulary beside it)."""
    def kas(width, heads, kv, d, ff, experts, top, eff, vocab):
        att = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv, dim=d, vdim=d, scale=d ** -0.5,
                                                q_temp=dict(coef=0.1, every=256)))
        left = dict(heads=heads // 2, kv_heads=kv, dim=d, vdim=d, conv=4, scale=d ** -0.5, rot=dict(base=10000.0, dims=d // 2))
        right = dict(heads=heads // 2, dim=d, vdim=d, decay=[1.0 - 2.0 ** (-5 - 0.4 * i) for i in range(heads // 2)])
        par = dict(type="parallel", mixer=dict(left=left, right=right))
        dense = dict(kind="dense", ff=ff)
        moe = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=eff))
        layers = [dict(att, mlp=dense), dict(par, mlp=moe), dict(par, mlp=dense), dict(att, mlp=moe), dict(par, mlp=moe),
                  dict(par, mlp=dense)]
        return dict(architecture="Kasarax", width=width, vocab=vocab, norm=dict(eps=1e-6), logit_scale=0.5, layers=layers)

    if name == "w2048":      # 16 heads of 128 (2 key/value heads), halves of 8 heads; 32 experts of 2,048, 4 chosen
        return kas(2048, 16, 2, 128, 8192, 32, 4, 2048, 32768), mepatar_sizes(name)[0]
    if name == "w1024":      # 8 heads of 128 (2 key/value heads), halves of 4 heads; 16 experts of 1,024, 4 chosen
        return kas(1024, 8, 2, 128, 4096, 16, 4, 1024, 32768), mepatar_sizes(name)[0]
    raise ValueError(name)


def kasarax_decode_bytes(cfg, batch, context):
    """Bytes a decode step has to read or write: the weights of every layer (of the experts, those that `batch`
    tokens can reach at most), the head, and what the live requests keep: the attention caches as far back as the
    context, the lightning states in 32-bit (read and written) and the convolutions' tails."""
    W, V = cfg["width"], cfg["vocab"]
    total = V * W * 2

    def attention(m, bias):
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        D = -(-max(d, dv) // 16) * 16
        return ((H + G) * d + G * dv + (H if bias else 0)) * W * 2 + W * H * dv * 2 + batch * context * G * 2 * D * 2

    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "attention":
            total += attention(m, True)
        else:
            a, r = m["left"], m["right"]
            total += attention(a, False)
            total += batch * (a.get("conv", 1) - 1) * ((a["heads"] + a["kv_heads"]) * a["dim"] + a["kv_heads"] * a["vdim"]) * 4 * 2
            H, d, dv = r["heads"], r["dim"], r["vdim"]
            total += (2 * H * d + 2 * H * dv) * W * 2 + W * H * dv * 2 + batch * H * d * dv * 4 * 2
        f = L["mlp"]
        if f and f["kind"] == "dense":
            total += 3 * f["ff"] * W * 2
        elif f:
            r, e = f["router"], f["expert"]
            total += r["experts"] * W * 4 + min(r["experts"], batch * r["top"]) * 2 * e["ff"] * W * 2
    return total


def kasarax_prefill_flops(cfg, T):
    """FLOPs of one prompt of T tokens by the design's own arithmetic: products, the chosen experts, causal
    attention, and the lightning states' updates and read-outs (4 d dv per head and token)."""
    W, V = cfg["width"], cfg["vocab"]
    total = 2 * V * W
    pairs = T * (T + 1) // 2

    def attention(m, gate):
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        return 2 * T * (((H + G) * d + G * dv + (H if gate else 0)) * W + W * H * dv) + H * 2 * (d + dv) * pairs

    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "attention":
            total += attention(m, True)
        else:
            r = m["right"]
            H, d, dv = r["heads"], r["dim"], r["vdim"]
            total += attention(m["left"], False) + 2 * T * ((2 * H * d + 2 * H * dv) * W + W * H * dv) + T * H * 4 * d * dv
        f = L["mlp"]
        if f and f["kind"] == "dense":
            total += 2 * T * 3 * f["ff"] * W
        elif f:
            total += 2 * T * (f["router"]["experts"] * W + f["router"]["top"] * 2 * f["expert"]["ff"] * W)
    return total


def run_kasarax(args):
    """Prefill and decode throughput of Kasarax at layer sizes of real models (random weights), beside Mepatar
    (the framework's closest design: a mixer and a feed-forward side by side on one stream, attention and matrix
    states, routed experts) at equal width, number of layers and vocabulary.  One JSON line per model and size."""
    import numpy as np
    import torch
    from railgun_b200.engine.batch import StepEntry
    from railgun_b200.engine.engine import Engine
    page, pool_tokens = 16, 64 * 4096
    pk, pk_src = peaks()
    for size in (args.sizes.split(",") if args.sizes else ["w1024", "w2048"]):
        for label, cfg in zip(("kasarax", "mepatar"), kasarax_sizes(size)):
            mdir = model_folder(cfg)
            eng = Engine(mdir, dtype="bfloat16", block_size=page, num_gpu_blocks=pool_tokens // page, max_num_seqs=64,
                         max_num_batched_tokens=8192, max_model_len=4096)
            runner = eng.runner
            V = cfg["vocab"]
            rng = np.random.default_rng(0)
            _, _, time_decode = decode_tools(runner, V, rng)
            line = {"mode": "kasarax", "size": size, "model": label, "layer_runs": len(runner.model.order),
                    "cache_bytes_per_token": runner.cache.bytes_per_token()}
            for b in (8, 64):
                tok_s, ms, n_launch, _ = time_decode(b, args.steps, args.warmup, 1000 * b, args.context)
                line[f"decode_b{b}_tok_s"], line[f"decode_b{b}_ms"] = round(tok_s, 1), round(ms, 4)
                line[f"decode_b{b}_launches_per_step"] = n_launch // args.steps
                ctx = args.context + args.warmup + args.steps // 2
                by = kasarax_decode_bytes(cfg, b, ctx) if label == "kasarax" else mepatar_decode_bytes(cfg, b, ctx)
                line[f"decode_b{b}_GB_per_step"] = round(by / 1e9, 3)
                line[f"decode_b{b}_frac_hbm"] = round(by / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)
            prompt = rng.integers(0, V, size=args.tokens).tolist()
            times = []
            for i in range(args.warmup + 7):
                torch.cuda.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                runner.step([StepEntry(7000 + i, prompt, [args.tokens - 1])])
                t1.record()
                torch.cuda.synchronize()
                runner.end([7000 + i])
                times.append(t0.elapsed_time(t1))
            runner.check_device_errors()
            ms = sorted(times[args.warmup:])[len(times[args.warmup:]) // 2]
            fl = kasarax_prefill_flops(cfg, args.tokens) if label == "kasarax" else mepatar_prefill_flops(cfg, args.tokens)
            line.update(prefill_tokens=args.tokens, prefill_ms=round(ms, 3), prefill_tok_s=round(args.tokens / ms * 1e3, 1),
                        prefill_TFLOP=round(fl / 1e12, 3), prefill_frac_flops=round(fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3),
                        peaks=pk_src)
            print(json.dumps(line), flush=True)
            del eng, runner, time_decode
            torch.cuda.empty_cache()
    return 0


def run_kernels(args):
    """Times the hot kernels one by one, each as a CUDA graph of 16 calls over 16 different operand sets (so
    that weights and caches come from HBM, not L2), with CUDA events around replays.  One JSON line per case."""
    import torch
    from railgun_b200 import ops
    dev, L = "cuda:0", 16
    cfg = LLAMA_3_2_1B
    H, I, nh, nkv, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    QKV, page = (nh + 2 * nkv) * d, 16

    def timed(fn, reps=20):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            g.replay()
        t1.record()
        torch.cuda.synchronize()
        ops.tc_gemm_check()
        return t0.elapsed_time(t1) / reps * 1e3 / L          # microseconds per call

    def weights(n, k):
        return [(torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16) for _ in range(L)]

    def out(case, us, **more):
        print(json.dumps(dict(case=case, us=round(us, 2), **more)), flush=True)

    want = set(args.cases.split(",")) if args.cases else None
    on = lambda name: want is None or name in want

    if on("decode_gemm"):
        for M in (1, 8):
            x = torch.randn(M, H, device=dev).to(torch.bfloat16)
            xi = torch.randn(M, I, device=dev).to(torch.bfloat16)
            resid, nw = torch.randn(M, H, device=dev), torch.ones(H, device=dev)
            for name, n, k, silu in (("qkv", QKV, H, False), ("o", H, H, False), ("gate_up", 2 * I, H, True), ("down", H, I, False)):
                ws = weights(n, k)
                inp = xi if k == I else x
                us = timed(lambda: [ops.skinny_gemm(inp, w, silu_mul=silu) for w in ws])
                us_lib = timed(lambda: [torch.mm(inp, w.t()) for w in ws])
                more = {}
                if name in ("o", "down"):
                    more["residual_epilogue_us"] = round(timed(lambda: [ops.skinny_gemm_residual(inp, w, resid, nw, 1e-5) for w in ws]), 2)
                else:
                    rows = ops.skinny_gemm_residual(x, weights(H, H)[0], resid, nw, 1e-5)
                    more["norm_finishing_us"] = round(timed(lambda: [ops.skinny_gemm_scaled(rows, w, silu_mul=silu) for w in ws]), 2)
                out(f"decode product {name} M{M} ({n} x {k})", us, GBs=round(n * k * 2 / us / 1e3, 1), cublas_us=round(us_lib, 2), **more)
    if on("decode_gemm_mid"):
        # decode batches of 17 to 64 rows: the swapped-operand tcgen05 product against the library
        for M in (32, 64):
            x = torch.randn(M, H, device=dev).to(torch.bfloat16)
            xi = torch.randn(M, I, device=dev).to(torch.bfloat16)
            for name, n, k, silu in (("qkv", QKV, H, False), ("o", H, H, False), ("gate_up", 2 * I, H, True), ("down", H, I, False)):
                ws = weights(n, k)
                inp = xi if k == I else x
                res = {}
                for sp in (0, 1, 2, 4, 8):
                    res[f"splits{sp}"] = round(timed(lambda: [ops.tc_stream_gemm(inp, w, silu_mul=silu, splits=sp) for w in ws]), 2)
                us_lib = timed(lambda: [ops.silu_mul(torch.mm(inp, w.t()), interleaved=True) if silu else torch.mm(inp, w.t()) for w in ws])
                out(f"decode product {name} M{M} ({n} x {k})", res["splits0"], GBs=round(n * k * 2 / res["splits0"] / 1e3, 1),
                    cublas_us=round(us_lib, 2), **res)
    if on("decode_attention"):
        for B, ctx in ((1, 1024), (8, 1024), (64, 1024), (8, 8192)):
            blocks = -(-ctx // page)
            kvs = [torch.randn(B * blocks, 2, nkv, page, d, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(B * blocks, dtype=torch.int32, device=dev).view(B, blocks).contiguous()
            q = torch.randn(B, QKV, device=dev).to(torch.bfloat16)
            o = torch.empty(B, nh * d, dtype=torch.bfloat16, device=dev)
            req = torch.arange(B, dtype=torch.int32, device=dev)
            pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
            splits = ops.decode_splits(B, nkv, ctx)
            us = timed(lambda: [ops.decode_attention(q, QKV, o, kv, bt, None, B, req, pos, nh, nkv, d, 0, d ** -0.5, splits)
                                for kv in kvs])
            more = {}
            if 2 <= splits <= 8:     # beside the engine's way (a second kernel adds the splits): the splits as a cluster
                more["cluster_us"] = round(timed(lambda: [ops.decode_attention(
                    q, QKV, o, kv, bt, None, B, req, pos, nh, nkv, d, 0, d ** -0.5, splits, cluster=True) for kv in kvs]), 2)
            out(f"decode attention B{B} ctx{ctx} splits{splits}", us, GBs=round(B * ctx * nkv * d * 4 / us / 1e3, 1), **more)
    if on("sampling"):
        V = cfg["vocab_size"]
        for rows in (8, 64):
            logits = [torch.randn(rows, V, device=dev) * 9.0 for _ in range(L)]      # peaked rows, as a trained model's
            seed = torch.arange(rows, dtype=torch.int64, device=dev)
            counter = torch.zeros(rows, dtype=torch.int64, device=dev)
            res = {"argmax": round(timed(lambda: [ops.argmax(l) for l in logits]), 1)}
            for name, T, k, p in (("temperature", 0.8, 0, 1.0), ("top_k_50", 0.8, 50, 1.0), ("top_p_0.9", 0.8, 0, 0.9),
                                  ("top_k_50_top_p_0.9", 0.8, 50, 0.9), ("top_k_2000", 0.8, 2000, 1.0)):
                t = torch.full((rows,), T, device=dev)
                kk = torch.full((rows,), k, dtype=torch.int32, device=dev)
                pp = torch.full((rows,), p, device=dev)
                res[name] = round(timed(lambda: [ops.sample(l, t, kk, pp, seed, counter) for l in logits]), 1)
            out(f"sampling {rows} rows x {V} logits", res["temperature"], **res)
    if on("prefill_gemm"):
        for M in (2048, 8192):
            x = torch.randn(M, H, device=dev).to(torch.bfloat16)
            xi = torch.randn(M, I, device=dev).to(torch.bfloat16)
            for name, n, k, silu in (("qkv", QKV, H, False), ("o", H, H, False), ("gate_up", 2 * I, H, True), ("down", H, I, False)):
                ws = weights(n, k)
                inp = xi if k == I else x
                fl = 2 * M * n * k
                res = {}
                for tile in ops.TC_TILES:
                    us = timed(lambda: [ops.tc_gemm(inp, w, silu_mul=silu, tile=tile) for w in ws])
                    res[tile] = f"{us:.1f} us, {fl / us / 1e6:.0f} TFLOP/s"
                us_lib = timed(lambda: [ops.silu_mul(torch.mm(inp, w.t()), interleaved=True) if silu else torch.mm(inp, w.t()) for w in ws])
                out(f"prefill product {name} M{M} ({n} x {k})", us_lib, cublas_TFLOPs=round(fl / us_lib / 1e6), **res)
    if on("primitives"):
        # cycles of the building blocks of the tcgen05 kernels (per warp instruction and scheduler, per MMA, per wait)
        print(json.dumps({"case": "sm_100a primitives, cycles", **ops.probe_sm100(dev)}), flush=True)
    if on("prefill_attention"):
        for T in (2048, 8192):
            blocks = -(-T // page)
            kvs = [torch.randn(blocks, 2, nkv, page, d, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(blocks, dtype=torch.int32, device=dev).view(1, blocks).contiguous()
            q = torch.randn(T, QKV, device=dev).to(torch.bfloat16)
            o = torch.empty(T, nh * d, dtype=torch.bfloat16, device=dev)
            pos = torch.arange(T, dtype=torch.int32, device=dev)
            t128 = torch.tensor([(k, min(128, T - k), 0) for k in range(0, T, 128)], dtype=torch.int32, device=dev)
            t64 = torch.tensor([(k, min(64, T - k), 0) for k in range(0, T, 64)], dtype=torch.int32, device=dev)
            fl = nh * 4 * d * T * (T + 1) / 2
            us = timed(lambda: [ops.prefill_attention_tc(q, o, kv, bt, t128, pos, nh, nkv, d, 0, d ** -0.5) for kv in kvs])
            us2 = timed(lambda: [ops.prefill_attention(q, QKV, o, kv, bt, t64, pos, nh, nkv, d, 0, d ** -0.5) for kv in kvs])
            out(f"prefill attention T{T} tcgen05", us, TFLOPs=round(fl / us / 1e6, 1), mma_sync_us=round(us2, 2))
    if on("latent_attention"):
        # attention over the latent cache (16 heads, latent 512 + 64) beside the dense model's kernels at equal
        # width; decode: bytes of cache read per second, prompts: FLOP/s of the products the kernel does
        pk, _ = peaks()
        Hh, R, dr = 16, 512, 64
        D = R + dr
        for B, ctx in ((8, 1024), (64, 1024), (8, 8192)):
            blocks = -(-ctx // page)
            caches = [torch.randn(B * blocks, page, D, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(B * blocks, dtype=torch.int32, device=dev).view(B, blocks).contiguous()
            qa = torch.randn(B, Hh, D, device=dev).to(torch.bfloat16)
            o = torch.empty(B, Hh, R, dtype=torch.bfloat16, device=dev)
            req = torch.arange(B, dtype=torch.int32, device=dev)
            pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
            sp = ops.latent_decode_splits(B, 1, ctx)
            us = timed(lambda: [ops.latent_attention_mma(qa, o, c, bt, None, None, B, req, pos, R, 0, D ** -0.5, sp) for c in caches])
            kvs = [torch.randn(B * blocks, 2, nkv, page, d, device=dev).to(torch.bfloat16) for _ in range(L)]
            q = torch.randn(B, QKV, device=dev).to(torch.bfloat16)
            o2 = torch.empty(B, nh * d, dtype=torch.bfloat16, device=dev)
            sp2 = ops.decode_splits(B, nkv, ctx)
            us2 = timed(lambda: [ops.decode_attention(q, QKV, o2, kv, bt, None, B, req, pos, nh, nkv, d, 0, d ** -0.5, sp2) for kv in kvs])
            gbs, gbs2 = B * ctx * D * 2 / us / 1e3, B * ctx * nkv * d * 4 / us2 / 1e3
            out(f"latent decode attention B{B} ctx{ctx} splits{sp}", us, GBs=round(gbs, 1), frac=round(gbs / pk["hbm_gbs"], 3),
                llama_us=round(us2, 2), llama_GBs=round(gbs2, 1), llama_frac=round(gbs2 / pk["hbm_gbs"], 3))
        for T in (2048, 8192):
            blocks = -(-T // page)
            caches = [torch.randn(blocks, page, D, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(blocks, dtype=torch.int32, device=dev).view(1, blocks).contiguous()
            qa = torch.randn(T, Hh, D, device=dev).to(torch.bfloat16)
            o = torch.empty(T, Hh, R, dtype=torch.bfloat16, device=dev)
            pos = torch.arange(T, dtype=torch.int32, device=dev)
            req = torch.zeros(T, dtype=torch.int32, device=dev)
            t64 = torch.tensor([(k, min(64, T - k), 0) for k in range(0, T, 64)], dtype=torch.int32, device=dev)
            us = timed(lambda: [ops.latent_attention_mma(qa, o, c, bt, t64, None, t64.shape[0], req, pos, R, 0, D ** -0.5) for c in caches])
            fl = Hh * 2 * (D + R) * T * (T + 1) / 2
            kvs = [torch.randn(blocks, 2, nkv, page, d, device=dev).to(torch.bfloat16) for _ in range(L)]
            q = torch.randn(T, QKV, device=dev).to(torch.bfloat16)
            o2 = torch.empty(T, nh * d, dtype=torch.bfloat16, device=dev)
            t128 = torch.tensor([(k, min(128, T - k), 0) for k in range(0, T, 128)], dtype=torch.int32, device=dev)
            fl2 = nh * 4 * d * T * (T + 1) / 2
            us2 = timed(lambda: [ops.prefill_attention_tc(q, o2, kv, bt, t128, pos, nh, nkv, d, 0, d ** -0.5) for kv in kvs])
            us3 = timed(lambda: [ops.prefill_attention(q, QKV, o2, kv, bt, t64, pos, nh, nkv, d, 0, d ** -0.5) for kv in kvs])
            out(f"latent prompt attention T{T}", us, TFLOPs=round(fl / us / 1e6, 1), frac=round(fl / us / 1e6 / pk["bf16_tflops"], 3),
                llama_tcgen05_us=round(us2, 2), llama_tcgen05_TFLOPs=round(fl2 / us2 / 1e6, 1),
                llama_tcgen05_frac=round(fl2 / us2 / 1e6 / pk["bf16_tflops"], 3),
                llama_mma_sync_us=round(us3, 2), llama_mma_sync_TFLOPs=round(fl2 / us3 / 1e6, 1))
    if on("talking_attention"):
        # talking-heads attention (heads x key/value heads x key size = value size) on the tensor cores beside the
        # dense model's kernels at equal width: single tokens by bytes of cache read, prompts by the design's own
        # FLOPs (scores and values once per head and key, and the mixing of the heads' scores)
        from types import SimpleNamespace
        pk, _ = peaks()
        for Hh, G, dd in ((16, 2, 128), (8, 2, 64)):
            R, D, hpg = G * dd, 2 * G * dd, Hh // G
            for B, ctx in ((8, 1024), (64, 1024)):
                blocks = -(-ctx // page)
                caches = [torch.randn(B * blocks, page, D, device=dev).to(torch.bfloat16) for _ in range(L)]
                bt = torch.arange(B * blocks, dtype=torch.int32, device=dev).view(B, blocks).contiguous()
                qa = torch.randn(B, Hh, D, device=dev).to(torch.bfloat16)
                o = torch.empty(B, Hh * dd, dtype=torch.bfloat16, device=dev)
                req = torch.arange(B, dtype=torch.int32, device=dev)
                pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
                sp = ops.latent_decode_splits(B, 1, ctx)
                us = timed(lambda: [ops.latent_attention_mma(qa, o, c, bt, None, None, B, req, pos, R, 0, 1.0, sp,
                                                             select=(dd, hpg), score_from=R) for c in caches])
                kvs = [torch.randn(B * blocks, 2, nkv, page, d, device=dev).to(torch.bfloat16) for _ in range(L)]
                q = torch.randn(B, QKV, device=dev).to(torch.bfloat16)
                o2 = torch.empty(B, nh * d, dtype=torch.bfloat16, device=dev)
                sp2 = ops.decode_splits(B, nkv, ctx)
                us2 = timed(lambda: [ops.decode_attention(q, QKV, o2, kv, bt, None, B, req, pos, nh, nkv, d, 0, d ** -0.5, sp2) for kv in kvs])
                gbs, gbs2 = B * ctx * D * 2 / us / 1e3, B * ctx * nkv * d * 4 / us2 / 1e3
                out(f"talking decode attention H{Hh} G{G} d{dd} B{B} ctx{ctx}", us, GBs=round(gbs, 1),
                    frac=round(gbs / pk["hbm_gbs"], 3), llama_us=round(us2, 2), llama_GBs=round(gbs2, 1),
                    llama_frac=round(gbs2 / pk["hbm_gbs"], 3))
            T = 2048
            blocks = -(-T // page)
            caches = [torch.randn(blocks, page, D, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(blocks, dtype=torch.int32, device=dev).view(1, blocks).contiguous()
            qa = torch.randn(T, Hh, D, device=dev).to(torch.bfloat16)
            qc = torch.randn(T, Hh, G * dd, device=dev).to(torch.bfloat16)
            o = torch.empty(T, Hh * dd, dtype=torch.bfloat16, device=dev)
            pos = torch.arange(T, dtype=torch.int32, device=dev)
            req = torch.zeros(T, dtype=torch.int32, device=dev)
            t64 = torch.tensor([(k, min(64, T - k), 0) for k in range(0, T, 64)], dtype=torch.int32, device=dev)
            us_rows = timed(lambda: [ops.latent_attention_mma(qa, o, c, bt, t64, None, t64.shape[0], req, pos, R, 0, 1.0,
                                                              select=(dd, hpg), score_from=R) for c in caches])
            batch = SimpleNamespace(cu_seqlens=torch.tensor([0, T], dtype=torch.int32, device=dev),
                                    context_lens=torch.tensor([T], dtype=torch.int32, device=dev), prefill_tiles=t64,
                                    positions=pos, req_of_token=req)
            ops.TALKING_FLASH_MAX_KEYS, kept = 256, ops.TALKING_FLASH_MAX_KEYS        # time both forms at every size
            us_flash = timed(lambda: [ops.talking_prefill_flash(qc, c, bt, batch, G, dd, dd, o) for c in caches])
            ops.TALKING_FLASH_MAX_KEYS = kept
            fl = (Hh * 4 * dd + 2 * Hh * Hh) * T * (T + 1) / 2
            kvs = [torch.randn(blocks, 2, nkv, page, d, device=dev).to(torch.bfloat16) for _ in range(L)]
            q = torch.randn(T, QKV, device=dev).to(torch.bfloat16)
            o2 = torch.empty(T, nh * d, dtype=torch.bfloat16, device=dev)
            t128 = torch.tensor([(k, min(128, T - k), 0) for k in range(0, T, 128)], dtype=torch.int32, device=dev)
            fl2 = nh * 4 * d * T * (T + 1) / 2
            us2 = timed(lambda: [ops.prefill_attention_tc(q, o2, kv, bt, t128, pos, nh, nkv, d, 0, d ** -0.5) for kv in kvs])
            us3 = timed(lambda: [ops.prefill_attention(q, QKV, o2, kv, bt, t64, pos, nh, nkv, d, 0, d ** -0.5) for kv in kvs])
            out(f"talking prompt attention H{Hh} G{G} d{dd} T{T}", min(us_rows, us_flash), rows_form_us=round(us_rows, 2),
                flash_form_us=round(us_flash, 2), TFLOPs=round(fl / min(us_rows, us_flash) / 1e6, 1),
                frac=round(fl / min(us_rows, us_flash) / 1e6 / pk["bf16_tflops"], 3),
                llama_tcgen05_us=round(us2, 2), llama_tcgen05_frac=round(fl2 / us2 / 1e6 / pk["bf16_tflops"], 3),
                llama_mma_sync_us=round(us3, 2), llama_mma_sync_frac=round(fl2 / us3 / 1e6 / pk["bf16_tflops"], 3))
    if on("rupulix_rows"):
        # the memory kernels of the hyper-connected stream and of the recurrence, by bytes they have to move, beside
        # the dense model's residual-add + RMSNorm kernel
        from types import SimpleNamespace
        pk, _ = peaks()
        W, S, C, K, Bk = 2048, 2, 2048, 4, 8
        for T in (8, 2048):
            cps = [torch.randn(T, S, W, device=dev) for _ in range(L)]
            ys = [torch.randn(T, W, device=dev).to(torch.bfloat16) for _ in range(L)]
            mix, oc, ic, nw = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(S, device=dev), torch.ones(W, device=dev)
            us = timed(lambda: [ops.hyper_step(c, None, y, mix, oc, ic, nw, 1e-6, torch.bfloat16) for c, y in zip(cps, ys)])
            by = T * W * (8 * S + 2 + 2)
            rs = [torch.randn(T, W, device=dev) for _ in range(L)]
            us2 = timed(lambda: [ops.add_rmsnorm(r, y, nw, 1e-6, torch.bfloat16) for r, y in zip(rs, ys)])
            by2 = T * W * (8 + 2 + 2)
            out(f"hyper step S{S} W{W} T{T}", us, GBs=round(by / us / 1e3, 1), frac=round(by / us / 1e3 / pk["hbm_gbs"], 3),
                add_rmsnorm_us=round(us2, 2), add_rmsnorm_frac=round(by2 / us2 / 1e3 / pk["hbm_gbs"], 3))
            R_ = 1 if T > 8 else T
            per = T // R_
            batch = SimpleNamespace(cu_seqlens=torch.arange(0, T + 1, per, dtype=torch.int32, device=dev),
                                    req_of_token=(torch.arange(T, device=dev) // per).to(torch.int32),
                                    start_pos=torch.zeros(R_, dtype=torch.int32, device=dev),
                                    state_slots=torch.arange(R_, dtype=torch.int32, device=dev), max_query_len=per)
            projs = [torch.randn(T, 2 * C, device=dev).to(torch.bfloat16) for _ in range(L)]
            vec = lambda n: torch.randn(n, device=dev) * 0.1
            xb, yb, cb, rb, ib, lam = vec(C), vec(C), vec(C), vec(C), vec(C), vec(C) - 3.0
            taps = torch.randn(C, K, device=dev) * 0.3
            state = torch.zeros(R_, K, C, device=dev)
            wg = torch.randn(Bk, C // Bk, 2 * C // Bk, device=dev) * 0.05
            us_c = timed(lambda: [ops.recurrent_conv(p, C, xb, taps, cb, state, batch) for p in projs])
            us_ = [ops.recurrent_conv(p, C, xb, taps, cb, state, batch) for p in projs]
            us_g = timed(lambda: [torch.bmm(u.view(-1, Bk, C // Bk).transpose(0, 1), wg) for u in us_])
            gs = [torch.bmm(u.view(-1, Bk, C // Bk).transpose(0, 1), wg) for u in us_]
            # the same products from u as two bfloat16 numbers (what portions of a bfloat16 model run)
            hv = [ops.recurrent_conv(p, C, xb, taps, cb, state, batch, halves_blocks=Bk)[1] for p in projs]
            wh = torch.cat([wg.to(torch.bfloat16)] * 2, dim=1).contiguous()
            us_h = timed(lambda: [torch.bmm(h.view(-1, Bk, 2 * C // Bk).transpose(0, 1), wh, out_dtype=torch.float32) for h in hv])
            us_s = timed(lambda: [ops.recurrent_scan(p, 0, C, yb, xb, u, g, rb, ib, lam, 8.0, state, batch)
                                  for p, u, g in zip(projs, us_, gs)])
            by_c, by_s = T * C * (2 + 4), T * C * (4 + 8 + 2 + 2)
            out(f"recurrence C{C} blocks{Bk} taps{K} T{T}", us_c + us_g + us_s, conv_us=round(us_c, 2),
                conv_frac=round(by_c / us_c / 1e3 / pk["hbm_gbs"], 3), gates_product_us=round(us_g, 2),
                gates_TFLOPs=round(2 * T * C * 2 * (C // Bk) / us_g / 1e6, 2), gates_product_bf16_halves_us=round(us_h, 2), scan_us=round(us_s, 2),
                scan_frac=round(by_s / us_s / 1e3 / pk["hbm_gbs"], 3))
    if on("mepatar_rows"):
        # Mepatar's own kernels by the bytes they have to move (and, for the matrix states, the 32-bit work they
        # have to do), each beside the like kernel of another design: the norm in groups beside add + RMSNorm, the
        # input convolution beside the recurrence's convolution, the state scans beside the recurrence's scan,
        # attention that keeps the first tokens beside the same kernel with a plain window
        from types import SimpleNamespace
        pk, _ = peaks()
        fp32_tflops = 148 * 128 * 2 * 1.9e9 / 1e12          # FMA lanes x 2 x the clock under load
        W, Hh, Hq, dd, K, G = 2048, 16, 8, 128, 4, 2
        for T in (64, 4096):
            R_ = 1 if T > 64 else T
            per = T // R_
            batch = SimpleNamespace(cu_seqlens=torch.arange(0, T + 1, per, dtype=torch.int32, device=dev),
                                    num_requests=R_, req_of_token=(torch.arange(T, device=dev) // per).to(torch.int32),
                                    start_pos=torch.full((R_,), 1000, dtype=torch.int32, device=dev),
                                    state_slots=torch.arange(R_, dtype=torch.int32, device=dev), max_query_len=per,
                                    positions=(1000 + torch.arange(T, device=dev) % per).to(torch.int32))
            rs = [torch.randn(T, W, device=dev) for _ in range(L)]
            ys = [torch.randn(T, W, device=dev).to(torch.bfloat16) for _ in range(L)]
            nw, nw2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
            us = timed(lambda: [ops.add_group_rmsnorm(r, y, [nw, nw2], 4, 1e-6, torch.bfloat16) for r, y in zip(rs, ys)])
            us2 = timed(lambda: [ops.add_rmsnorm(r, y, nw, 1e-6, torch.bfloat16) for r, y in zip(rs, ys)])
            by, by2 = T * W * (8 + 2 + 4), T * W * (8 + 2 + 2)
            out(f"norm in 4 groups, two outputs W{W} T{T}", us, frac=round(by / us / 1e3 / pk["hbm_gbs"], 3),
                add_rmsnorm_us=round(us2, 2), add_rmsnorm_frac=round(by2 / us2 / 1e3 / pk["hbm_gbs"], 3))
            taps = torch.randn(K, W, device=dev) * 0.3
            cstate = [torch.randn(R_, K - 1, W, device=dev) for _ in range(L)]
            us = timed(lambda: [(ops.causal_conv(y, 0, taps, c, batch, torch.bfloat16, residual=True),
                                 ops.conv_state_update(y, 0, c, batch)) for y, c in zip(ys, cstate)])
            by = T * W * (2 + 2) + R_ * (K - 1) * W * 8
            out(f"input convolution taps{K} W{W} T{T}", us, frac=round(by / us / 1e3 / pk["hbm_gbs"], 3))
            qs = [torch.randn(T, Hq * dd, device=dev) * 0.1 for _ in range(L)]
            ks = [torch.nn.functional.normalize(torch.randn(T, Hq, dd, device=dev), dim=-1).view(T, Hq * dd) for _ in range(L)]
            vs = [torch.randn(T, Hh * dd, device=dev).to(torch.bfloat16) for _ in range(L)]
            sts = [torch.zeros(R_, Hh, dd, dd, device=dev) for _ in range(L)]      # [slots, H, dv, d]
            gg, bb = torch.rand(T, Hh, device=dev) * 0.1 + 0.9, torch.rand(T, Hh, device=dev)
            decay = torch.full((Hh,), 0.99, device=dev)
            q16 = [torch.randn(T, Hh * dd, device=dev) * 0.1 for _ in range(L)]
            k16 = [torch.randn(T, Hh * dd, device=dev) * 0.1 for _ in range(L)]
            us_r = timed(lambda: [ops.state_scan(q, k, v, st, batch, Hh, dd, dd, decay=decay)
                                  for q, k, v, st in zip(q16, k16, vs, sts)])
            us_d = timed(lambda: [ops.state_scan(q, k, v, st, batch, Hh, dd, dd, g=gg, beta=bb)
                                  for q, k, v, st in zip(qs, ks, vs, sts)])
            by_r = T * (2 * Hh * dd * 4 + Hh * dd * (2 + 4)) + R_ * Hh * dd * dd * 8
            by_d = T * (2 * Hq * dd * 4 + Hh * dd * (2 + 4)) + R_ * Hh * dd * dd * 8
            out(f"state scans H{Hh} d{dd} dv{dd} T{T} ({R_} requests)", us_r + us_d, retention_us=round(us_r, 2),
                retention_frac_hbm=round(by_r / us_r / 1e3 / pk["hbm_gbs"], 3),
                retention_frac_fp32=round(T * Hh * 6 * dd * dd / us_r / 1e6 / fp32_tflops, 3), delta_us=round(us_d, 2),
                delta_frac_hbm=round(by_d / us_d / 1e3 / pk["hbm_gbs"], 3),
                delta_frac_fp32=round(T * Hh * 6 * dd * dd / us_d / 1e6 / fp32_tflops, 3))
            os_ = [torch.randn(T, Hh, dd, device=dev) for _ in range(L)]
            us = timed(lambda: [ops.head_norm_gate(o, v, nw[:dd], 1e-6, torch.bfloat16) for o, v in zip(os_, vs)])
            by = T * Hh * dd * (4 + 2 + 2)
            out(f"heads' norm and gate H{Hh} dv{dd} T{T}", us, frac=round(by / us / 1e3 / pk["hbm_gbs"], 3))
        # attention over a window of 512 that keeps the first 4 tokens: 64 single tokens at context 4,096, and a prompt
        for T, B in ((64, 64), (4096, 1)):
            ctx = 4096
            blocks = -(-ctx // page)
            kvs = [torch.randn(B * blocks, 2, G, page, dd, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(B * blocks, dtype=torch.int32, device=dev).view(B, blocks).contiguous()
            q = (torch.randn(T, Hh * dd, device=dev) * dd ** -0.5).to(torch.bfloat16)
            req = (torch.arange(T, device=dev) // (T // B)).to(torch.int32)
            pos = (torch.arange(T, device=dev) % (T // B) + (ctx - T // B)).to(torch.int32)
            o = torch.empty(T, Hh * dd, dtype=torch.bfloat16, device=dev)
            res = {}
            for keep in (4, 0):
                if B > 1:
                    splits = ops.decode_splits(T, G * (-(-(Hh // G) // 8)), 512 + keep)
                    res[keep] = timed(lambda: [ops.decode_attention(q, Hh * dd, o, kv, bt, None, T, req, pos, Hh, G, dd, 512, 1.0,
                                                                    splits, keep_first=keep) for kv in kvs])
                else:
                    t64 = torch.tensor([(k, min(64, T - k), 0) for k in range(0, T, 64)], dtype=torch.int32, device=dev)
                    res[keep] = timed(lambda: [ops.prefill_attention(q, Hh * dd, o, kv, bt, t64, pos, Hh, G, dd, 512, 1.0,
                                                                     keep_first=keep) for kv in kvs])
            seen = sum(min(int(p) + 1, 516) for p in pos.tolist())
            by = (B * 516 * G * 2 * dd * 2) if B > 1 else 0
            fl = Hh * 4 * dd * seen
            out(f"attention window 512 keeping 4, H{Hh} G{G} d{dd}, {B} requests x {T // B} tokens", res[4],
                plain_window_us=round(res[0], 2), TFLOPs=round(fl / res[4] / 1e6, 2),
                **({"frac_hbm": round(by / res[4] / 1e3 / pk["hbm_gbs"], 3), "plain_window_frac_hbm": round(
                    (B * 512 * G * 2 * dd * 2) / res[0] / 1e3 / pk["hbm_gbs"], 3)} if B > 1 else
                   {"frac_flops": round(fl / res[4] / 1e6 / pk["bf16_tflops"], 3)}))
    if on("kasarax_rows"):
        # Kasarax's own kernels by the bytes they have to move, each beside the like kernel of another design: the sum
        # of two normed branches beside the norm in groups, the per-token work before attention with norms over the
        # whole of q and k beside the per-head norms, attention with a sink and a gate per head beside the same
        # kernels without, the norm over all lightning heads beside the per-head norm, the experts' rows times
        # their weights beside the plain gather
        from types import SimpleNamespace
        pk, _ = peaks()
        W, Hh, dd, G, K = 2048, 16, 128, 2, 4
        Hl = Hh // 2
        from railgun_b200.parts.latent_attention import rotary_frequencies
        freq = rotary_frequencies(dd // 2, 10000.0).to(dev)
        for T in (64, 4096):
            R_ = 1 if T > 64 else T
            per = T // R_
            batch = SimpleNamespace(cu_seqlens=torch.arange(0, T + 1, per, dtype=torch.int32, device=dev),
                                    num_requests=R_, req_of_token=(torch.arange(T, device=dev) // per).to(torch.int32),
                                    start_pos=torch.full((R_,), 1000, dtype=torch.int32, device=dev),
                                    state_slots=torch.arange(R_, dtype=torch.int32, device=dev), max_query_len=per,
                                    positions=(1000 + torch.arange(T, device=dev) % per).to(torch.int32))
            ya = [torch.randn(T, W, device=dev).to(torch.bfloat16) for _ in range(L)]
            yb = [torch.randn(T, W, device=dev).to(torch.bfloat16) for _ in range(L)]
            rs = [torch.randn(T, W, device=dev) for _ in range(L)]
            nw, nw2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
            us = timed(lambda: [ops.norm_sum([a, b], [nw, nw2], [0.5, 0.5], 1e-6) for a, b in zip(ya, yb)])
            us2 = timed(lambda: [ops.add_group_rmsnorm(r, y, [nw, nw2], 4, 1e-6, torch.bfloat16) for r, y in zip(rs, ya)])
            by, by2 = T * W * (2 + 2 + 4), T * W * (8 + 2 + 4)
            out(f"sum of two normed branches W{W} T{T}", us, frac=round(by / us / 1e3 / pk["hbm_gbs"], 3),
                group_norm_us=round(us2, 2), group_norm_frac=round(by2 / us2 / 1e3 / pk["hbm_gbs"], 3))
            # the left half: convolution with its state update, then norms over the whole of q and k, rotation, cache write
            C = (Hl + G) * dd + G * dd
            projs = [torch.randn(T, C, device=dev).to(torch.bfloat16) for _ in range(L)]
            taps = torch.randn(K, C, device=dev) * 0.3
            cstate = [torch.randn(R_, K - 1, C, device=dev) for _ in range(L)]
            us = timed(lambda: [(ops.causal_conv(y, 0, taps, c, batch, torch.float32), ops.conv_state_update(y, 0, c, batch))
                                for y, c in zip(projs, cstate)])
            by = T * C * (2 + 4) + R_ * (K - 1) * C * 8
            out(f"convolution on q, k, v taps{K} C{C} T{T}", us, frac=round(by / us / 1e3 / pk["hbm_gbs"], 3))
            convd = [torch.randn(T, C, device=dev) for _ in range(L)]
            blocks = -(-T // page) + 1
            kvc = [torch.zeros(blocks, 2, G, page, dd, dtype=torch.bfloat16, device=dev) for _ in range(L)]
            slots = torch.arange(T, dtype=torch.int32, device=dev)
            qn, kn, qn1 = torch.ones(Hl * dd, device=dev), torch.ones(G * dd, device=dev), torch.ones(dd, device=dev)
            fac = torch.full((Hl,), 0.1, device=dev)
            us = timed(lambda: [ops.attention_prepare(x, kv, qn, kn, 1e-6, freq, dd // 2, True, batch.positions, slots, fac,
                                                      Hl, G, dd, dd, dd, norm_whole=True, out_dtype=torch.bfloat16)
                                for x, kv in zip(convd, kvc)])
            us2 = timed(lambda: [ops.attention_prepare(x, kv, qn1, qn1, 1e-6, freq, dd // 2, True, batch.positions, slots,
                                                       fac, Hl, G, dd, dd, dd) for x, kv in zip(projs, kvc)])
            by, by2 = T * C * (4 + 2), T * C * (2 + 2)
            out(f"before attention, norms over all of q and k, H{Hl} G{G} d{dd} T{T}", us,
                frac=round(by / us / 1e3 / pk["hbm_gbs"], 3), per_head_us=round(us2, 2),
                per_head_frac=round(by2 / us2 / 1e3 / pk["hbm_gbs"], 3))
            # the right half: silu on q, k, v; the norm over all heads with a sigmoid gate
            pr = [torch.randn(T, 4 * Hl * dd, device=dev).to(torch.bfloat16) for _ in range(L)]
            f0 = rotary_frequencies(0, 10.0).to(dev)
            us = timed(lambda: [ops.retention_prepare(x, 0, Hl * dd, f0, 0, batch.positions, Hl, dd, 1.0, silu=True,
                                                      v_off=2 * Hl * dd, dv=dd) for x in pr])
            fd = rotary_frequencies(dd, 10000.0).to(dev)
            us2 = timed(lambda: [ops.retention_prepare(x, 0, Hl * dd, fd, dd, batch.positions, Hl, dd, 0.1) for x in pr])
            by, by2 = T * 3 * Hl * dd * (2 + 4), T * 2 * Hl * dd * (2 + 4)
            out(f"lightning prepare (silu on q, k, v) H{Hl} d{dd} T{T}", us, frac=round(by / us / 1e3 / pk["hbm_gbs"], 3),
                retention_us=round(us2, 2), retention_frac=round(by2 / us2 / 1e3 / pk["hbm_gbs"], 3))
            os_ = [torch.randn(T, Hl, dd, device=dev) for _ in range(L)]
            gs = [torch.randn(T, Hl * dd, device=dev).to(torch.bfloat16) for _ in range(L)]
            nwl = torch.ones(Hl * dd, device=dev)
            us = timed(lambda: [ops.head_norm_gate(o, g, nwl, 1e-6, torch.bfloat16, whole=True, gate_kind="sigmoid")
                                for o, g in zip(os_, gs)])
            us2 = timed(lambda: [ops.head_norm_gate(o, g, nwl[:dd], 1e-6, torch.bfloat16) for o, g in zip(os_, gs)])
            by = T * Hl * dd * (4 + 2 + 2)
            out(f"norm over all heads and sigmoid gate H{Hl} dv{dd} T{T}", us, frac=round(by / us / 1e3 / pk["hbm_gbs"], 3),
                per_head_us=round(us2, 2), per_head_frac=round(by / us2 / 1e3 / pk["hbm_gbs"], 3))
            # the experts' rows, each times its weight, in expert order, beside the plain gather
            E, top = 32, 4
            xs = [torch.randn(T, W, device=dev).to(torch.bfloat16) for _ in range(L)]
            ids = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(T)]).to(torch.int32).contiguous()
            wts = torch.rand(T, top, device=dev)
            sp, pp, tiles = ops.moe_align(ids, E, 128 if T > 64 else 32)
            us = timed(lambda: [ops.moe_scaled_rows(x, sp, top, wts, T * top) for x in xs])
            by = T * top * W * (2 + 2)
            out(f"experts' rows times their weights W{W} T{T} top{top}", us, frac=round(by / us / 1e3 / pk["hbm_gbs"], 3))
        # causal attention with a sink and a gate per head beside the same kernels without: 64 single tokens at
        # context 4,096, and a prompt of 4,096
        for T, B in ((64, 64), (4096, 1)):
            ctx = 4096
            blocks = -(-ctx // page)
            kvs = [torch.randn(B * blocks, 2, G, page, dd, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(B * blocks, dtype=torch.int32, device=dev).view(B, blocks).contiguous()
            q = (torch.randn(T, Hh * dd, device=dev) * dd ** -0.5).to(torch.bfloat16)
            req = (torch.arange(T, device=dev) // (T // B)).to(torch.int32)
            pos = (torch.arange(T, device=dev) % (T // B) + (ctx - T // B)).to(torch.int32)
            o = torch.empty(T, Hh * dd, dtype=torch.bfloat16, device=dev)
            sink = torch.zeros(Hh, device=dev)
            gate = torch.randn(T, Hh, device=dev).to(torch.bfloat16)
            res = {}
            for with_sink in (True, False):
                more = dict(sink=sink, gate=gate) if with_sink else {}
                if B > 1:
                    splits = ops.decode_splits(T, G * (-(-(Hh // G) // 8)), ctx)
                    res[with_sink] = timed(lambda: [ops.decode_attention(q, Hh * dd, o, kv, bt, None, T, req, pos, Hh, G, dd, 0,
                                                                         1.0, splits, **more) for kv in kvs])
                else:
                    t64 = torch.tensor([(k, min(64, T - k), 0) for k in range(0, T, 64)], dtype=torch.int32, device=dev)
                    res[with_sink] = timed(lambda: [ops.prefill_attention(q, Hh * dd, o, kv, bt, t64, pos, Hh, G, dd, 0, 1.0,
                                                                          **more) for kv in kvs])
            seen = sum(int(p) + 1 for p in pos.tolist())
            by = B * ctx * G * 2 * dd * 2
            fl = Hh * 4 * dd * seen
            out(f"attention with a sink and a gate, H{Hh} G{G} d{dd}, {B} requests x {T // B} tokens", res[True],
                without_us=round(res[False], 2), TFLOPs=round(fl / res[True] / 1e6, 2),
                **({"frac_hbm": round(by / res[True] / 1e3 / pk["hbm_gbs"], 3),
                    "without_frac_hbm": round(by / res[False] / 1e3 / pk["hbm_gbs"], 3)} if B > 1 else
                   {"frac_flops": round(fl / res[True] / 1e6 / pk["bf16_tflops"], 3),
                    "without_frac_flops": round(fl / res[False] / 1e6 / pk["bf16_tflops"], 3)}))
    if on("moe"):
        # the routed experts' two grouped products (32 experts of 1,024 at width 2,048, 4 choices) beside the dense
        # model's gate|up and down products of equal work: decode by bytes of weights read, prompts by FLOP/s
        pk, _ = peaks()
        E, F, top = 32, 1024, 4
        for T in (8, 64, 2048, 8192):
            x = torch.randn(T, H, device=dev).to(torch.bfloat16)
            wgu = [(torch.randn(E, 2 * F, H, device=dev) / H ** 0.5).to(torch.bfloat16) for _ in range(L)]
            wd = [(torch.randn(E, H, F, device=dev) / F ** 0.5).to(torch.bfloat16) for _ in range(L)]
            ids = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(T)]).to(torch.int32).contiguous()
            rows = ops.moe_tile_rows(x.dtype, T * top, E, H, F)
            sp, pp, tiles = ops.moe_align(ids, E, rows)
            act = ops.moe_grouped_gemm(x, sp, top, wgu[0], tiles, T * top, True, rows)
            us1 = timed(lambda: [ops.moe_grouped_gemm(x, sp, top, w, tiles, T * top, True, rows) for w in wgu])
            us2 = timed(lambda: [ops.moe_grouped_gemm(act, None, 1, w, tiles, T * top, False, rows) for w in wd])
            touched = int(torch.unique(ids).numel())
            fl = 2 * T * top * 3 * F * H
            by = touched * 3 * F * H * 2
            # the dense products of equal work: an intermediate size of top * F
            I2 = top * F
            w1 = weights(2 * I2, H)
            w2 = weights(H, I2)
            xi = torch.randn(T, I2, device=dev).to(torch.bfloat16)
            if T <= 16:
                d1 = timed(lambda: [ops.skinny_gemm(x, w, silu_mul=True) for w in w1])
                d2 = timed(lambda: [ops.skinny_gemm(xi, w) for w in w2])
            else:
                d1 = timed(lambda: [ops.silu_mul(torch.mm(x, w.t()), interleaved=True) for w in w1])
                d2 = timed(lambda: [torch.mm(xi, w.t()) for w in w2])
            dby = 3 * I2 * H * 2
            out(f"routed experts T{T} ({E} x {F}, top {top}, tiles of {rows})", us1 + us2, gate_up_us=round(us1, 2),
                down_us=round(us2, 2), GBs=round(by / (us1 + us2) / 1e3, 1), TFLOPs=round(fl / (us1 + us2) / 1e6, 1),
                frac_hbm=round(by / (us1 + us2) / 1e3 / pk["hbm_gbs"], 3),
                frac_flops=round(fl / (us1 + us2) / 1e6 / pk["bf16_tflops"], 3),
                dense_us=round(d1 + d2, 2), dense_GBs=round(dby / (d1 + d2) / 1e3, 1),
                dense_TFLOPs=round(fl / (d1 + d2) / 1e6, 1), dense_frac_hbm=round(dby / (d1 + d2) / 1e3 / pk["hbm_gbs"], 3),
                dense_frac_flops=round(fl / (d1 + d2) / 1e6 / pk["bf16_tflops"], 3))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the named configuration (0: all)")
    ap.add_argument("--mode", default="all", choices=["all", "decode", "prefill", "kernels", "dizatar", "rupulix", "mepatar", "kasarax"],
                    help="all: the contract's line; decode / prefill: one short measurement (for profiling); "
                         "kernels: the hot kernels one by one; dizatar / rupulix: prefill and decode of the Dizatar / Rupulix design at "
                         "layer sizes of real models beside the dense model of equal width; mepatar: the same for "
                         "the Mepatar design beside Rupulix; kasarax: the same for the Kasarax design beside Mepatar")
    ap.add_argument("--sizes", default="", help="--mode dizatar / rupulix / mepatar / kasarax: comma-separated subset of w1024, w2048")
    ap.add_argument("--cases", default="", help="--mode kernels: comma-separated subset of sampling, decode_gemm, "
                    "decode_gemm_mid, decode_attention, prefill_gemm, prefill_attention, primitives, latent_attention, moe, "
                    "talking_attention, rupulix_rows, mepatar_rows, kasarax_rows")
    ap.add_argument("--batch", type=int, default=8, help="--mode decode: requests in the batch")
    ap.add_argument("--tokens", type=int, default=PREFILL_TOKENS, help="--mode prefill: prompt length")
    ap.add_argument("--context", type=int, default=CONTEXT, help="--mode decode: tokens each request holds")
    ap.add_argument("--windows", type=int, default=0, help="--mode decode: 1 times three windows only (for profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace on the candle crates: pip finds neither setup.py nor "
                          "pyproject.toml, and cargo/rustc are not installed"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.mode == "kernels":
        return run_kernels(args)
    if args.mode == "dizatar":
        return run_dizatar(args)
    if args.mode == "rupulix":
        return run_rupulix(args)
    if args.mode == "mepatar":
        return run_mepatar(args)
    if args.mode == "kasarax":
        return run_kasarax(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())

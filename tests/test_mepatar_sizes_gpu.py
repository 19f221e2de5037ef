"""Mepatar at the layer sizes the benchmark times (8 heads of 128 x 128 at width 1,024; fewer and smaller experts,
a small vocabulary, three layers), against the plain statement: the 32-bit path held tightly; bfloat16 (the scan
with 16 rows of S per thread, the tensor-core attention kernels at head size 128 with a window and kept tokens,
the grouped tcgen05 product followed by the clamped activation) by the loose rule for positions whose routing is
near a tie."""
import numpy as np
import pytest

import helpers
import mepatar_cases as C
import plain_mepatar as P

pytestmark = pytest.mark.gpu

CASE_W = dict(
    architecture="Mepatar", width=1024, vocab=512, norm=dict(eps=1e-6, groups=4), embedding=dict(scale=32.0),
    canon=dict(taps=4),
    layers=[C.layer(C.retention(8, 128, 128, [1.0 - 2.0 ** (-5 - 0.4 * i) for i in range(8)], dims=128), C.dense(2048)),
            C.layer(C.delta(8, 4, 128, 128, 4), C.moe(8, 2, 512, 7.0)),
            C.layer(C.attention(8, 2, 128, 128, dims=64, window=100, keep=4), C.moe(8, 2, 512, 7.0))])
LENGTHS = [330, 40, 197, 3]
_state: dict = {}


def setup(tmp_factory):
    if not _state:
        # small weights: rows of 1,024 numbers must not saturate the activations
        folder = tmp_factory.mktemp("mepatar_W")

        def shrink(t):
            for k in t:
                if t[k].ndim == 2 and not k.endswith(".conv") and "canon" not in k and k != "embed":
                    t[k] *= 0.25
        C.write_model(CASE_W, 17, folder, change=shrink)
        plain = C.Plain(folder)
        reqs = {f"r{i}": p for i, p in enumerate(C.prompts(CASE_W["vocab"], LENGTHS, seed=31))}
        logits, margins = {}, {}
        for k, v in reqs.items():
            m = []
            logits[k] = P.forward(v, plain.w, plain.cfg, margins=m)
            margins[k] = np.min(np.stack(m), axis=0)
        _state.update(dir=folder, reqs=reqs, logits=logits, margins=margins)
    return _state


def run(st, dtype, steps, out_dir):
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    runner = ModelRunner(st["dir"], dtype=dtype, page_size=16, max_tokens=helpers.peak_tokens(steps, 64), max_requests=4)
    rp = Replayer(runner, out_dir)
    for s in steps:
        rp.feed(s)
    runner.check_device_errors()
    runner.alloc.check()
    return helpers.collect(steps, out_dir, CASE_W["vocab"])


@pytest.mark.parametrize("mode", ["whole", "tail", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_sizes_match_plain(dtype, mode, tmp_path, tmp_path_factory):
    st = setup(tmp_path_factory)
    reqs = st["reqs"]
    steps = {"whole": lambda: helpers.trace_whole(reqs), "tail": lambda: helpers.trace_tail_decode(reqs, 120),
             "mixed": lambda: helpers.trace_mixed(reqs, max_live=4, seed=3, sizes=(70, 1, 2, 33, 1, 130, 1, 5))}[mode]()
    rows = run(st, dtype, steps, tmp_path)
    tight, loose = (5e-5, 5e-5) if dtype == "float32" else (6e-2, 0.7)
    over = held = 0
    for name, toks in reqs.items():
        ref = st["logits"][name]
        scale = np.abs(ref).max()
        for p in range(len(toks)):
            err = np.abs(rows[(name, p)] - ref[p]).max() / scale
            clear = dtype == "float32" or st["margins"][name][p] >= 0.03
            held += clear
            assert err <= loose, f"{dtype} {mode}: request {name} position {p}: relative error {err:.3e}"
            over += bool(clear and err > tight)
    assert held >= 0.1 * sum(LENGTHS) and over <= 1 + 0.02 * held, f"{dtype} {mode}: {over} of {held} over {tight}"

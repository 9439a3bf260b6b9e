"""The Zerusun design in the engine against the plain implementation (GPU): every mechanism alone, whole prompts, cuts
down to two tokens, decoding, unequal batches, pages and state slots used again, keys far away, at page borders and
either side of a window's edge, the first token in a state hundreds of tokens later, other sizes than any real model's,
and greedy generation through the entry point and the scheduler."""
import copy
import os

import numpy as np
import pytest

from plain import zerusun_plain as P
from zerusun_helpers import (CONFIG_A, CONFIG_B, CONFIG_C, bf16_round, config, dense, draw_weights, latent, lightning, make_folder, moe,
                             steady_choice, tokens)

pytestmark = pytest.mark.gpu

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def f64(w):
    return {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


class Models:
    """Per configuration and dtype: (folder, config, weights for the plain implementation).  The float32 runs read
    weights stored in 32 bits with routers left free; the bfloat16 runs read the same values stored as bfloat16 with
    routers whose choice is fixed (a rounding of the router's input must not change the chosen set)."""

    def __init__(self, factory):
        self.items = {}
        for i, (name, cfg) in enumerate(CONFIGS.items()):
            w = draw_weights(cfg, 500 + i)
            self.items[name, "float32"] = (make_folder(factory.mktemp(f"zs_{name}_f32"), cfg, w, "F32"), cfg, f64(w))
            ws = steady_choice(cfg, w, i)
            self.items[name, "bfloat16"] = (make_folder(factory.mktemp(f"zs_{name}_bf16"), cfg, ws, "BF16"), cfg, f64(ws))

    def __getitem__(self, key):
        return self.items[key if isinstance(key, tuple) else (key, "float32")]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return Models(tmp_path_factory)


def engine_for(folder, dtype, **kw):
    from purhie_b200.engine import Engine
    opts = dict(page_size=8, max_tokens=512, max_requests=4, poison_cache=True)
    opts.update(kw)
    return Engine.from_folder(folder, dtype=dtype, **opts)


def close(got, ref, tol):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape
    assert np.isfinite(got).all()
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err < tol, f"relative error {err:.3e} (allowed {tol:.1e})"


def run_cut(engine, rid, toks, cuts):
    """Feed ``toks`` in portions of the given sizes (the last portion takes what is left); all logits."""
    from purhie_b200.engine import StepEntry
    engine.add_request(rid)
    rows, at = [], 0
    for n in list(cuts) + [len(toks)]:
        n = min(n, len(toks) - at)
        if n <= 0:
            break
        rows.append(engine.step([StepEntry(rid, toks[at:at + n], list(range(n)))]))
        at += n
    engine.release(rid)
    return np.concatenate(rows)


def part_of(cfg, layer, name):
    from purhie_b200.config import ModelConfig
    spec = ModelConfig.from_dict(cfg).model_spec()
    part = spec["layers"][layer]["parts"][name] if layer is not None else spec[name]
    return part["kind"], part["params"]


def mixer_in_pieces(p, x, pieces, request=1):
    p.add_request(request)
    out, at = [], 0
    for n in pieces:
        out.append(p.mixer_step([(request, n)], x[at:at + n]))
        at += n
    p.release(request)
    return np.concatenate(out)


# ---- whole models ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_cuts_and_decoding_agree_with_the_plain_implementation(models, name, dtype):
    folder, cfg, w = models[name, dtype]
    eng = engine_for(folder, dtype)
    toks = tokens(75, cfg["vocab"], 7)
    ref = P.forward(cfg, w, toks)
    whole = run_cut(eng, "whole", toks, [])
    close(whole, ref, TOL[dtype])
    # one token (the first of a sequence alone), then two, then portions of changing size, single tokens between them
    cut = run_cut(eng, "cut", toks, [1, 2, 2, 5, 1, 1, 16, 3, 17, 2, 1])
    close(cut, ref, TOL[dtype])
    # a prompt, then token by token: every decode step replays a graph
    tail = run_cut(eng, "tail", toks, [30] + [1] * 45)
    close(tail, ref, TOL[dtype])
    if dtype == "float32":                      # the 32-bit kernels add in one order however the tokens arrive
        assert np.abs(cut - whole).max() <= 1e-5 * np.abs(ref).max()
        assert np.abs(tail - whole).max() <= 1e-5 * np.abs(ref).max()
    eng.check_cache()
    eng.close()


def test_every_layer_run_agrees_with_the_plain_implementation(models):
    """The residual stream after each layer run, the repeated ones each time, so that a fault shows where it starts."""
    from purhie_b200.config import ModelConfig
    from purhie_b200.engine import StepEntry
    for name in ("A", "B"):
        folder, cfg, w = models[name]
        toks = tokens(40, cfg["vocab"], 3)
        ref = []
        P.forward(cfg, w, toks, ref)
        schedule = ModelConfig.from_dict(cfg).model_spec()["schedule"]
        runs = [i for i, c in enumerate(schedule) if c["layer"] < len(cfg["layers"])]      # the others are reinjections
        assert len(runs) == len(ref)
        eng = engine_for(folder, "float32")
        got = {}
        eng.set_layer_dump(lambda entry, x: got.__setitem__(entry, np.array(x)))
        eng.add_request("x")
        eng.step([StepEntry("x", toks, [len(toks) - 1])])
        assert sorted(got) == list(range(len(schedule)))
        for entry, r in zip(runs, ref):
            close(got[entry], r, 1e-4)
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(models, name, dtype):
    from purhie_b200.engine import StepEntry
    folder, cfg, w = models[name, dtype]
    # room for two requests' states and about 100 tokens: five requests must take turns, pages come back poisoned
    eng = engine_for(folder, dtype, max_tokens=104, max_requests=2)
    lengths = [41, 9, 1, 56, 23]
    reqs = {f"r{i}": tokens(n, cfg["vocab"], 20 + i) for i, n in enumerate(lengths)}
    refs = {r: P.forward(cfg, w, t) for r, t in reqs.items()}
    at = {r: 0 for r in reqs}
    got = {r: [] for r in reqs}
    waiting, live, step = list(reqs), [], 0
    portions = [2, 7, 1, 1, 13, 2, 1, 5, 1, 1, 1, 9]
    while waiting or live:
        while waiting and len(live) < 2:
            r = waiting.pop(0)
            eng.add_request(r)
            live.append(r)
        entries = []
        for j, r in enumerate(live):
            n = min(portions[(step + 3 * j) % len(portions)], len(reqs[r]) - at[r])
            entries.append(StepEntry(r, reqs[r][at[r]:at[r] + n], list(range(n))))
        out = eng.step(entries)
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.request_id].append(out[row:row + n])
            row += n
            at[e.request_id] += n
        for r in list(live):
            if at[r] == len(reqs[r]):
                eng.release(r)
                live.remove(r)
        step += 1
        eng.check_cache()
    for r in reqs:
        close(np.concatenate(got[r]), refs[r], TOL[dtype])
    eng.close()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16"), ("C", "float32")])
def test_a_long_prompt_alone_and_beside_a_decode_row_and_a_two_token_portion(models, name, dtype):
    """330 tokens: many windows, hundreds of steps of the recurrence (in chunks), and enough (token, choice) pairs for
    the experts' tiled products."""
    from purhie_b200.engine import StepEntry
    folder, cfg, w = models[name, dtype]
    eng = engine_for(folder, dtype, max_tokens=1024)
    toks = tokens(330, cfg["vocab"], 11)
    ref = P.forward(cfg, w, toks)
    close(run_cut(eng, "whole", toks, []), ref, TOL[dtype])
    eng.add_request("a"); eng.add_request("b"); eng.add_request("c")
    eng.step([StepEntry("b", toks[:5], []), StepEntry("c", toks[:9], [])])
    out = eng.step([StepEntry("b", toks[5:6], [0]), StepEntry("a", toks[:300], list(range(300))), StepEntry("c", toks[9:11], [0, 1])])
    close(out[1:301], ref[:300], TOL[dtype])
    close(out[:1], ref[5:6], TOL[dtype])
    close(out[301:], ref[9:11], TOL[dtype])
    eng.close()


def test_long_decoding_passes_many_windows_and_keeps_its_state(models):
    folder, cfg, w = models["A"]
    eng = engine_for(folder, "float32", max_tokens=256)
    toks = tokens(230, cfg["vocab"], 3)
    ref = P.forward(cfg, w, toks)
    got = run_cut(eng, "long", toks, [2] + [1] * 228)
    close(got, ref, TOL["float32"])
    eng.close()


def test_pages_that_every_window_has_passed_go_back_to_the_pool(tmp_path):
    """A model whose every layer looks back a few positions keeps only the pages that the next position can still see."""
    from purhie_b200.engine import StepEntry
    cfg = config(32, 30, [(latent(2, 8, 4, 8, 8, 12, 11), None), (latent(2, 8, 4, 8, 8, 12, 11), dense(24))], loop=(0, 1, 2))
    w = draw_weights(cfg, 1)
    folder = make_folder(tmp_path, cfg, w)
    eng = engine_for(folder, "float32", page_size=8, max_tokens=64)         # eight pages
    toks = tokens(200, cfg["vocab"], 2)
    ref = P.forward(cfg, f64(w), toks)
    eng.add_request("x")
    rows = []
    for at in range(0, 200, 10):                                             # 200 tokens through a pool of 64
        rows.append(eng.step([StepEntry("x", toks[at:at + 10], list(range(10)))]))
        assert min(eng.info()["free_pages"]) >= 8 - 4
        eng.check_cache()
    close(np.concatenate(rows), ref, TOL["float32"])
    eng.close()

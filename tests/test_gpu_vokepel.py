"""The Vokepel design in the engine against the plain implementation (GPU): every mechanism alone, whole prompts, cuts
down to two tokens, decoding, unequal batches, pages and state slots used again, keys far away, at page borders and
either side of a window's edge, a sink that shows, the first token in a state hundreds of tokens later, other sizes
than any real model's, and greedy generation through the entry point and the scheduler."""
import os

import numpy as np
import pytest

from plain import vokepel_plain as P
from vokepel_helpers import (CONFIG_A, CONFIG_B, CONFIG_C, bf16_round, config, dense, draw_weights, left_side, make_folder, pair, talking,
                             tokens)

pytestmark = pytest.mark.gpu

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def f64(w):
    return {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


class Models:
    """Per configuration and dtype: (folder, config, weights for the plain implementation); the same values stored in 32
    bits for the float32 runs and as bfloat16 for the others."""

    def __init__(self, factory):
        self.items = {}
        for i, (name, cfg) in enumerate(CONFIGS.items()):
            w = draw_weights(cfg, 700 + i)
            self.items[name, "float32"] = (make_folder(factory.mktemp(f"vk_{name}_f32"), cfg, w, "F32"), cfg, f64(w))
            self.items[name, "bfloat16"] = (make_folder(factory.mktemp(f"vk_{name}_bf16"), cfg, w, "BF16"), cfg, f64(w))

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
    for name in ("A", "B", "C"):
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
    """330 tokens: many windows and hundreds of steps of the recurrence, which then runs in chunks."""
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
    cfg = config(32, 30, [(talking(2, 1, 8, 11), None), (pair(left_side(2, 2, 8, 8, 11, 8), 16), dense(24))], loop=(0, 1, 2), mult=0.9)
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


# ---- every mechanism alone -------------------------------------------------------------------------------------------
def sharp_model(tmp, kind_m, width, seed, storage):
    """One mixer whose softmax is sharp (scores of a few units): a key more or less at a window's edge, or a sink left out,
    moves the output far beyond the tolerance."""
    cfg = config(width, 20, [(kind_m, None)])
    w = draw_weights(cfg, seed, std=0.5)
    return cfg, w, make_folder(tmp, cfg, w, storage)


# windows of 9 to 200 positions and none; groups of 1 to 6; one head alone (nobody to talk to) and thirty-two (above sixteen
# the tensor-core kernel takes a tile with a pair of CTAs); heads of 16, 32, 48, 64 and 96 take that kernel in bfloat16,
# the others the plain one
TALKERS = {
    "h4": (talking(4, 2, 16, 70, scale=2.0, softcap=8.0), 64),
    "h6": (talking(6, 2, 24, 33, scale=1.5, softcap=30.0), 48),
    "h12": (talking(12, 3, 8, 200, scale=3.0), 64),
    "h1": (talking(1, 1, 40, None, scale=1.0, softcap=2.0), 40),
    "h3": (talking(3, 3, 64, 9, scale=0.8, softcap=6.0), 24),
    "h5": (talking(5, 1, 32, 100, scale=1.2, softcap=10.0), 56),
    "h8": (talking(8, 2, 48, 45, scale=1.0), 72),
    "h16": (talking(16, 4, 96, 130, scale=0.7, softcap=12.0), 64),
    "h24": (talking(24, 4, 32, 75, scale=1.1, softcap=9.0), 48),
    "h32": (talking(32, 8, 16, 60, scale=1.6), 64),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(TALKERS))
def test_talking_attention_alone_whole_cut_decoded_and_batched(tmp_path, which, dtype):
    from purhie_b200.parts import PartProbe
    kind_m, width = TALKERS[which]
    cfg, w, folder = sharp_model(tmp_path, kind_m, width, 3, "F32" if dtype == "float32" else "BF16")
    m, eps = kind_m[1], cfg["norm"]["eps"]
    T = 260
    x = np.random.default_rng(1).normal(0, 1.0, (T, width)).astype(np.float32)
    if dtype == "bfloat16":
        x = bf16_round(x)
    wd = f64(w)
    ref = P.talking_attention(x.astype(np.float64), wd, "l0.mix.", m, eps)
    tol = 2e-4 if dtype == "float32" else 3e-2
    size = (m.get("mask") or {}).get("size")
    if size:      # the test can tell a window that is one position off
        for other in (size - 1, size + 1):
            off = P.talking_attention(x.astype(np.float64), wd, "l0.mix.", dict(m, mask={"size": other}), eps)
            assert np.abs(off - ref).max() > 3 * tol * np.abs(ref).max()
    # and a mixer that forgets the cap, the distance, or the talk between the heads
    assert np.abs(P.talking_attention(x.astype(np.float64), dict(wd, **{"l0.mix.r1": 0 * wd["l0.mix.r1"]}), "l0.mix.", m, eps) - ref).max() > 3 * tol * np.abs(ref).max()
    if m["heads"] > 1:
        assert np.abs(P.talking_attention(x.astype(np.float64), dict(wd, **{"l0.mix.talk": np.eye(m["heads"])}), "l0.mix.", m, eps) - ref).max() > 3 * tol * np.abs(ref).max()
    if m.get("softcap"):
        assert np.abs(P.talking_attention(x.astype(np.float64), wd, "l0.mix.", dict(m, softcap=None), eps) - ref).max() > 3 * tol * np.abs(ref).max()
    p = PartProbe("mixer", *part_of(cfg, 0, "mixer"), dtype=dtype)
    p.bind_folder(folder)
    p.mixer_cache(8, 80, 3)
    close(mixer_in_pieces(p, x, [T], 1), ref, tol)
    # portions down to two tokens and one, cut inside pages, windows and key blocks; then single tokens to the end
    close(mixer_in_pieces(p, x, [1, 2, 61, 2, 1, 1, 64, 37, 2, 30] + [1] * 59, 2), ref, tol)
    # two requests side by side, one decoding while the other brings a portion; pages of the first two are in use again
    p.add_request(3); p.add_request(4)
    a = p.mixer_step([(3, 150)], x[:150])
    both = p.mixer_step([(3, 1), (4, 90)], np.concatenate([x[150:151], x[:90]]))
    again = p.mixer_step([(4, 2), (3, 1)], np.concatenate([x[90:92], x[151:152]]))
    close(np.concatenate([a, both[:1], again[2:]]), ref[:152], tol)
    close(np.concatenate([both[1:], again[:2]]), ref[:92], tol)


# the left side alone: heads of 48, 64 and 128 (sizes the tensor-core kernel takes) and others; values narrower and wider
LEFTS = {
    "d64": (left_side(4, 1, 64, 64, 70, 32, base=300.0, scale=0.6), 64),
    "d128": (left_side(2, 1, 128, 128, 33, 128, base=1e4, scale=0.4), 48),
    "d24": (left_side(3, 3, 24, 40, 50, 2, base=2e5, scale=1.0), 64),
    "d16": (left_side(8, 2, 16, 8, None, 0, scale=1.2), 40),
    "d64v": (left_side(4, 4, 64, 32, 100, 16, base=77.0, scale=0.5), 40),
    "d48": (left_side(6, 2, 48, 48, 17, 48, base=1e3, scale=0.7), 72),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(LEFTS))
def test_attention_with_a_sink_alone_whole_cut_decoded_and_batched(tmp_path, which, dtype):
    from purhie_b200.parts import PartProbe
    left, width = LEFTS[which]
    cfg, w, folder = sharp_model(tmp_path, pair(left, 16), width, 4, "F32" if dtype == "float32" else "BF16")
    T = 260
    x = np.random.default_rng(2).normal(0, 1.0, (T, width)).astype(np.float32)
    if dtype == "bfloat16":
        x = bf16_round(x)
    wd = f64(w)
    ref = P.sink_attention(x.astype(np.float64), wd, "l0.mix.left.", left)
    tol = 2e-4 if dtype == "float32" else 3e-2
    size = (left.get("mask") or {}).get("size")
    if size:
        for other in (size - 1, size + 1):
            off = P.sink_attention(x.astype(np.float64), wd, "l0.mix.left.", dict(left, mask={"size": other}))
            assert np.abs(off - ref).max() > 3 * tol * np.abs(ref).max()
    # a softmax that leaves the sink out is far off, and one that counts it twice is told apart in 32 bits
    for other, bound in ((-1e30, tol), (np.log(2.0), 2e-4)):
        off = P.sink_attention(x.astype(np.float64), dict(wd, **{"l0.mix.left.sink": wd["l0.mix.left.sink"] + other}), "l0.mix.left.", left)
        assert np.abs(off - ref).max() > 3 * bound * np.abs(ref).max()
    kind, params = part_of(cfg, 0, "mixer")
    p = PartProbe("mixer", params["left"]["kind"], params["left"]["params"], dtype=dtype)
    p.bind_folder(folder)
    p.mixer_cache(8, 80, 3)
    close(mixer_in_pieces(p, x, [T], 1), ref, tol)
    close(mixer_in_pieces(p, x, [1, 2, 61, 2, 1, 1, 64, 37, 2, 30] + [1] * 59, 2), ref, tol)
    p.add_request(3); p.add_request(4)
    a = p.mixer_step([(3, 150)], x[:150])
    both = p.mixer_step([(3, 1), (4, 90)], np.concatenate([x[150:151], x[:90]]))
    again = p.mixer_step([(4, 2), (3, 1)], np.concatenate([x[90:92], x[151:152]]))
    close(np.concatenate([a, both[:1], again[2:]]), ref[:152], tol)
    close(np.concatenate([both[1:], again[:2]]), ref[:92], tol)


def far_key_case(storage, tmp, window=180, at=37):
    """A talking mixer, its weights and T input rows in which row `at` is built so that its first key head lines up with
    what the first head of every later query asks for: that key takes nearly all the weight of the rows that see it."""
    T = at + window + 6
    kind_m = talking(2, 2, 16, window, scale=6.0, softcap=40.0)
    cfg, w, folder = sharp_model(tmp, kind_m, 64, 5, storage)
    w["l0.mix.r1"] = np.zeros(2, dtype=np.float32)                                    # no pull toward near keys
    w["l0.mix.talk"] = np.eye(2, dtype=np.float32)
    folder = make_folder(tmp, cfg, w, storage)
    wd = f64(w)
    x = np.random.default_rng(2).normal(0, 1.0, (T, 64))
    x[at + 1:] = x[at + 1] * (1.0 + 0.01 * np.arange(T - at - 1))[:, None]          # later queries all ask for the same key
    q = x[at + 1] @ wd["l0.mix.q"].T
    x[at] = 3.0 * np.linalg.lstsq(wd["l0.mix.k"][:16], q[:16] / wd["l0.mix.k.norm"][:16], rcond=None)[0]
    x = bf16_round(x.astype(np.float32))
    return cfg, kind_m[1], wd, folder, x, T


def test_a_far_key_decides_the_output_just_inside_the_window_and_not_just_outside(tmp_path):
    from purhie_b200.parts import PartProbe
    window, at = 180, 37
    for dtype in ("float32", "bfloat16"):
        cfg, m, w, folder, x, T = far_key_case("F32" if dtype == "float32" else "BF16", tmp_path / dtype, window, at)
        ref = P.talking_attention(x.astype(np.float64), w, "l0.mix.", m, cfg["norm"]["eps"])
        edge = at + window                                                            # the first row that no longer sees `at`
        assert np.abs(ref[edge] - ref[edge - 1]).max() > 0.2 * np.abs(ref).max()       # the plain implementation shows the step
        p = PartProbe("mixer", *part_of(cfg, 0, "mixer"), dtype=dtype)
        p.bind_folder(folder)
        p.mixer_cache(8, 64, 2)
        tol = 2e-4 if dtype == "float32" else 4e-2
        close(mixer_in_pieces(p, x, [T], 1), ref, tol)
        close(mixer_in_pieces(p, x, [edge - 3] + [1] * (T - edge + 3), 2), ref, tol)   # the edge passes while decoding
        close(mixer_in_pieces(p, x, [edge - 1, 2, T - edge - 1], 1), ref, tol)         # and inside a two-token portion
        close(mixer_in_pieces(p, x, [at, 1, 7, T - at - 8], 2), ref, tol)              # the key alone in its step, on a page's slot 5


def test_the_recurrent_unit_alone_cut_batched_and_in_a_slot_used_again(models):
    from purhie_b200.parts import PartProbe
    for name, layer, dtype in (("A", 0, "float32"), ("A", 3, "float32"), ("B", 1, "float32"), ("C", 0, "bfloat16"), ("C", 2, "float32")):
        folder, cfg, w = models[name, dtype]
        rng = np.random.default_rng(layer)
        xs = {r: rng.normal(0, 1.0, (n, cfg["width"])).astype(np.float32) for r, n in ((1, 150), (2, 7), (3, 1), (4, 40))}
        if dtype == "bfloat16":
            xs = {r: bf16_round(x) for r, x in xs.items()}
        ref = {r: P.min_gru(x.astype(np.float64), w, f"l{layer}.mix.right.") for r, x in xs.items()}
        tol = 2e-4 if dtype == "float32" else 3e-2
        kind, params = part_of(cfg, layer, "mixer")
        p = PartProbe("mixer", params["right"]["kind"], params["right"]["params"], dtype=dtype)
        p.bind_folder(folder)
        p.mixer_cache(8, 16, 2)                                  # two state slots
        close(mixer_in_pieces(p, xs[1], [150], 1), ref[1], tol)                       # in chunks
        close(mixer_in_pieces(p, xs[1], [1, 2, 70, 2, 64, 11], 1), ref[1], tol)       # the slot again, zeroed; row by row
        close(mixer_in_pieces(p, xs[1], [3, 130, 17], 1), ref[1], tol)                # chunks that start from a state
        p.add_request(2); p.add_request(3)
        out = p.mixer_step([(2, 2), (3, 1)], np.concatenate([xs[2][:2], xs[3]]))
        rest = np.concatenate([p.mixer_step([(2, 1)], xs[2][i:i + 1]) for i in range(2, 7)])
        close(np.concatenate([out[:2], rest]), ref[2], tol)
        close(out[2:], ref[3], tol)
        p.release(3)
        p.add_request(4)
        a = p.mixer_step([(4, 3)], xs[4][:3])
        b = np.concatenate([p.mixer_step([(4, 1)], xs[4][i:i + 1]) for i in range(3, 40)])
        close(np.concatenate([a, b]), ref[4], tol)


def test_the_candidate_of_the_recurrent_unit_is_continuous_and_takes_both_branches():
    u = np.array([-3.0, -1e-9, 0.0, 1e-9, 2.5])
    c = P.min_gru_candidate(u)
    assert np.allclose(c, [1 / (1 + np.exp(3.0)), 0.5, 0.5, 0.5, 3.0], atol=1e-8)


def test_the_first_token_still_shows_hundreds_of_tokens_later_in_a_state_that_hardly_forgets(tmp_path):
    from purhie_b200.parts import PartProbe
    cfg = config(16, 10, [(pair(left_side(1, 1, 8, 8, 4, 0), 24), None)])
    w = draw_weights(cfg, 9)
    w["l0.mix.right.z.b"] = np.full(24, -7.0, dtype=np.float32)          # z near 1/1000: the state keeps what it has
    folder = make_folder(tmp_path, cfg, w)
    wd = f64(w)
    x = np.random.default_rng(4).normal(0, 1.0, (400, 16)).astype(np.float32)
    y = x.copy()
    wz = wd["l0.mix.right.z"]
    y[0] = 40.0 * wz.sum(axis=0) / np.linalg.norm(wz.sum(axis=0))          # a first token whose gates are wide open
    ref_x, ref_y = P.min_gru(x.astype(np.float64), wd, "l0.mix.right."), P.min_gru(y.astype(np.float64), wd, "l0.mix.right.")
    assert np.abs(ref_x[-1] - ref_y[-1]).max() > 0.1 * np.abs(ref_x).max()
    kind, params = part_of(cfg, 0, "mixer")
    p = PartProbe("mixer", params["right"]["kind"], params["right"]["params"])
    p.bind_folder(folder)
    p.mixer_cache(8, 8, 2)
    close(mixer_in_pieces(p, y, [1, 200] + [1] * 199, 1), ref_y, 2e-4)
    close(mixer_in_pieces(p, x, [400], 1), ref_x, 2e-4)


def test_the_two_sides_together_and_the_feed_forward_alone(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("A", 0), ("A", 3), ("B", 1), ("C", 2)):
        folder, cfg, w = models[name]
        m = cfg["layers"][layer]["mixer"]
        x = np.random.default_rng(layer).normal(0, 1.0, (90, cfg["width"])).astype(np.float32)
        ref = P.side_by_side(x.astype(np.float64), w, f"l{layer}.mix.", m)
        p = PartProbe("mixer", *part_of(cfg, layer, "mixer"))
        p.bind_folder(folder)
        p.mixer_cache(8, 40, 2)
        close(mixer_in_pieces(p, x, [90], 1), ref, 2e-4)
        close(mixer_in_pieces(p, x, [2, 1, 50, 2] + [1] * 35, 2), ref, 2e-4)
    for name, layer in (("A", 0), ("B", 2), ("C", 1)):
        folder, cfg, w = models[name]
        x = np.random.default_rng(layer).normal(0, 1.5, (37, cfg["width"])).astype(np.float32)
        ref = P.squared_relu_unit(x.astype(np.float64), w, f"l{layer}.mlp.")
        p = PartProbe("feed_forward", *part_of(cfg, layer, "feed_forward"))
        p.bind_folder(folder)
        close(p.feed_forward(x), ref, 2e-4)
        close(p.feed_forward(x[:1]), ref[:1], 2e-4)


def test_the_head_scales_and_caps_the_logits(models):
    from purhie_b200.parts import PartProbe
    for name in ("A", "B", "C"):
        folder, cfg, w = models[name]
        xn = np.random.default_rng(0).normal(0, 12.0, (5, cfg["width"])).astype(np.float32)
        y = xn.astype(np.float64) @ w["embed"].T * cfg.get("logit_scale", 1.0)
        ref = P.soft_cap(y, cfg["logit_softcap"]) if cfg.get("logit_softcap") else y
        if cfg.get("logit_softcap"):
            assert np.abs(y).max() > 1.2 * np.abs(ref).max()                 # the cap bites
        kind, params = part_of(cfg, None, "head")
        params = {k: v for k, v in params.items() if k != "tied_to"}          # alone, the head reads the table under its own name
        p = PartProbe("head", kind, dict(params, names={"weight": "embed"}))
        p.bind_folder(folder)
        close(p.head(xn, cfg["vocab"]), ref, 2e-4)


# ---- the tensor-core attention kernel inside whole models, its keys shared by several CTAs ---------------------------
def test_key_splits_of_the_tile_kernel_agree_with_the_plain_implementation(models):
    from purhie_b200.engine import StepEntry
    folder, cfg, w = models["C", "bfloat16"]
    toks = tokens(300, cfg["vocab"], 6)
    ref = P.forward(cfg, w, toks)
    for splits in (1, 3, 0):                                   # whole tiles, three CTAs a tile, the part's own choice
        eng = engine_for(folder, "bfloat16", max_tokens=1024, step_options={"tile16_splits": splits})
        close(run_cut(eng, "whole", toks, []), ref, TOL["bfloat16"])
        close(run_cut(eng, "tail", toks, [2, 250] + [1] * 48), ref, TOL["bfloat16"])
        eng.add_request("a"); eng.add_request("b")
        eng.step([StepEntry("a", toks[:200], [])])
        out = eng.step([StepEntry("a", toks[200:201], [0]), StepEntry("b", toks[:130], list(range(130)))])
        close(out[:1], ref[200:201], TOL["bfloat16"])
        close(out[1:], ref[:130], TOL["bfloat16"])
        eng.close()


def test_a_sink_survives_the_merges_of_the_tcgen05_and_tma_kernels(tmp_path):
    """Heads of 128 with a sink take the tcgen05 prompt kernel and the TMA decode kernel; with their keys shared between CTAs
    the sink joins the sum in the merge, once."""
    from purhie_b200.engine import StepEntry
    cfg = config(64, 40, [(pair(left_side(2, 1, 128, 128, 150, 64, base=1e4, scale=0.3), 32, 1.0, 0.2), dense(48)),
                          (pair(left_side(4, 2, 128, 128, None, 128, base=300.0, scale=0.2), 24, 0.9, 0.3), None)], mult=0.9)
    w = draw_weights(cfg, 12, std=0.5)
    for name in ("l0.mix.left.sink", "l1.mix.left.sink"):
        w[name] = w[name] + 3.0                                  # sinks that take a good part of the weight
    folder = make_folder(tmp_path, cfg, w, "BF16")
    toks = tokens(330, cfg["vocab"], 4)
    wd = f64(w)
    ref = P.forward(cfg, wd, toks)
    without = P.forward(cfg, dict(wd, **{n: wd[n] - 1e30 for n in ("l0.mix.left.sink", "l1.mix.left.sink")}), toks)
    assert np.abs(without - ref).max() > 3 * TOL["bfloat16"] * np.abs(ref).max()
    for options in ({}, {"decode_splits": 3, "prefill_splits": 2}, {"decode_splits": 8, "prefill_splits": 5}, {"sink_kernel": "tile"}):
        eng = engine_for(folder, "bfloat16", max_tokens=1024, step_options=options)
        close(run_cut(eng, "whole", toks, []), ref, TOL["bfloat16"])
        close(run_cut(eng, "tail", toks, [2, 270] + [1] * 58), ref, TOL["bfloat16"])
        eng.add_request("a"); eng.add_request("b")
        eng.step([StepEntry("a", toks[:200], [])])
        out = eng.step([StepEntry("a", toks[200:201], [0]), StepEntry("b", toks[:140], list(range(140)))])
        close(out[:1], ref[200:201], TOL["bfloat16"])
        close(out[1:], ref[:140], TOL["bfloat16"])
        eng.close()


# ---- generation -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "float32")])
def test_greedy_generation_through_the_entry_point_and_the_scheduler(models, name, dtype):
    from purhie_b200.api import load_model
    from purhie_b200.sampling import SamplerParams
    folder, cfg, w = models[name, dtype]
    model = load_model(folder, dtype=dtype)
    model.kv_cache_init(256, max_sequences=3, page_size=8, max_batch_tokens=24, prefill_chunk=11)
    prompts = [tokens(n, cfg["vocab"], 60 + i) for i, n in enumerate((1, 14, 37))]

    def plain_greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(P.forward(cfg, w, toks)[-1].argmax()))
        return toks[len(prompt):]
    expected = [plain_greedy(p, 10) for p in prompts]
    for p, exp in zip(prompts, expected):
        assert model.generate_ex(p, 10, SamplerParams.greedy()) == exp
    assert model.generate(prompts, max_new_tokens=10) == expected        # chunked prompts beside decoding requests
    model.free()


def test_the_command_line_generates_from_a_folder_of_this_design(models):
    import subprocess
    import sys
    from helpers import ROOT
    folder, cfg, w = models["B"]
    prompt = tokens(12, cfg["vocab"], 8)
    toks = list(prompt)
    for _ in range(5):
        toks.append(int(P.forward(cfg, w, toks)[-1].argmax()))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen_demo"), folder, ",".join(map(str, prompt)), "5", "--dtype", "float32",
                        "--ctx", "64"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert [int(x) for x in lines[2:7]] == toks[12:]


def test_trace_replay_reads_a_folder_of_this_design(models, tmp_path):
    from helpers import TraceRun
    folder, cfg, w = models["A"]
    toks = tokens(40, cfg["vocab"], 5)
    ref = P.forward(cfg, w, toks)
    run = TraceRun(folder, "float32", tmp_path, 128)
    run.vocab = cfg["vocab"]
    a = run.step(0, [("x", toks[:17], [0, 16])])
    b = run.step(1, [("x", toks[17:19], [1]), ("y", toks[:3], [2])])
    c = run.step(2, [("x", toks[19:], [20])], end=["x", "y"])
    run.close()
    close(np.concatenate([a.numpy(), b.numpy()[:1], c.numpy()]), ref[[0, 16, 18, 39]], TOL["float32"])
    close(b.numpy()[1:], ref[[2]], TOL["float32"])

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


# ---- every mechanism alone -------------------------------------------------------------------------------------------
def test_dynamic_tanh_norm_alone_with_and_without_an_addend(models):
    from purhie_b200.parts import PartProbe
    folder, cfg, w = models["A"]
    rng = np.random.default_rng(0)
    x = rng.normal(0, 2.0, (9, cfg["width"])).astype(np.float32)
    add = rng.normal(0, 1.0, (9, cfg["width"])).astype(np.float32)
    for layer, name, key in ((2, "norm", "l2.norm1"), (None, "final_norm", "final.norm")):
        p = PartProbe("norm", *part_of(cfg, layer, name))
        p.bind_folder(folder)
        stream, y = p.norm(x, add)
        close(stream, x.astype(np.float64) + add, 1e-6)
        close(y, P.dynamic_tanh(x.astype(np.float64) + add, w, key), 1e-5)
        close(p.norm(x)[1], P.dynamic_tanh(x.astype(np.float64), w, key), 1e-5)


def test_stretched_frequencies_follow_the_ramp_between_the_two_turn_counts():
    from purhie_b200.parts import PartProbe
    # no scaling; a ramp inside the pairs; a ramp whose ends fall outside them on both sides (lo clamped to 0, hi to dims - 1)
    for dims, base, scaling in ((12, 77.0, None), (16, 1e4, (8.0, 512, 32.0, 1.0)), (4, 500.0, (4.0, 64, 16.0, 2.0)), (6, 50.0, (16.0, 4096, 2000.0, 0.001))):
        kind, m = latent(2, 8, dims, 8, 8, 8, None, base=base, scaling=scaling)
        cfg = config(16, 10, [((kind, m), None)])
        pk, pp = part_of(cfg, 0, "mixer")
        pos = pp["position"]
        p = PartProbe("position", pos["kind"], dict(pos["params"], max_position=40))
        p.bind_random(0)
        table = p.position_table()                                         # [positions, cos | sin]
        f, stretch = P.rotary_frequencies(m["rot"])
        angle = np.arange(40)[:, None] * f[None, :]
        close(table[:, :dims // 2], np.cos(angle) * stretch, 1e-5)
        close(table[:, dims // 2:], np.sin(angle) * stretch, 1e-5)


def sharp_latent_model(tmp, kind_m, width, seed, storage):
    """One latent mixer whose softmax is sharp (scores of a few units): a key more or less at a window's edge moves the
    output far beyond the tolerance."""
    cfg = config(width, 20, [(kind_m, None)])
    w = draw_weights(cfg, seed, std=0.5)
    return cfg, w, make_folder(tmp, cfg, w, storage)


# rows of 128 + 32, 256 + 16 (five heads: tiles cut inside a token), 512 + 64 and 40 + 24 (padded) go through the tensor
# cores in bfloat16; 20 + 4 does not.  Windows of 70, 33 and 200 positions, and none.
LATENTS = {
    "c128": (latent(4, 16, 32, 24, 32, 128, 70, base=300.0, scale=0.35), 64),
    "c256": (latent(5, 16, 16, 8, 24, 256, 33, base=1e4, scaling=(4.0, 64, 16.0, 1.0), scale=0.25), 48),
    "c512": (latent(16, 8, 64, 8, 48, 512, 200, base=5e5, scale=0.2), 64),
    "c40": (latent(3, 24, 24, 16, 40, 40, None, base=50.0, scale=0.3), 40),
    "c20": (latent(2, 8, 4, 8, 12, 20, 9, base=20.0, scale=0.5), 24),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(LATENTS))
def test_latent_attention_alone_whole_cut_decoded_and_batched(tmp_path, which, dtype):
    from purhie_b200.parts import PartProbe
    kind_m, width = LATENTS[which]
    cfg, w, folder = sharp_latent_model(tmp_path, kind_m, width, 3, "F32" if dtype == "float32" else "BF16")
    m = kind_m[1]
    T = 260
    x = np.random.default_rng(1).normal(0, 1.0, (T, width)).astype(np.float32)
    if dtype == "bfloat16":
        x = bf16_round(x)
    ref = P.latent_attention_mixer(x.astype(np.float64), f64(w), "l0.mix.", m, cfg["norm"]["eps"])
    tol = 2e-4 if dtype == "float32" else 3e-2
    size = (m.get("mask") or {}).get("size")
    if size:      # the test can tell a window that is one position off
        for other in (size - 1, size + 1):
            off = P.latent_attention_mixer(x.astype(np.float64), f64(w), "l0.mix.", dict(m, mask={"size": other}), cfg["norm"]["eps"])
            assert np.abs(off - ref).max() > 3 * tol * np.abs(ref).max()
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


def far_key_case(dtype_storage, tmp, window=180, at=37, scale=0.3):
    """A latent mixer, its weights and T input rows in which row `at` is built so that its latent lines up with what the
    first head of every later query asks for: that key takes nearly all the weight of the rows that see it."""
    T = at + window + 6
    kind_m = latent(2, 16, 16, 16, 32, 32, window, base=1e4, scale=scale)
    cfg, w, folder = sharp_latent_model(tmp, kind_m, 64, 5, dtype_storage)
    wd = f64(w)
    x = np.random.default_rng(2).normal(0, 1.0, (T, 64))
    x[at + 1:] = x[at + 1] * (1.0 + 0.01 * np.arange(T - at - 1))[:, None]          # later queries all ask for the same latent
    q = (P.rms_norm(x[at + 1] @ wd["l0.mix.dq"].T, wd["l0.mix.dq.norm"], 1e-5) @ wd["l0.mix.uq"].T).reshape(2, 32)
    asked = q[0, :16] @ wd["l0.mix.uk"].reshape(2, 16, 32)[0]                        # head 0's query seen from the latent
    x[at] = np.linalg.lstsq(wd["l0.mix.dkv"][:32], asked / wd["l0.mix.dkv.norm"], rcond=None)[0]
    x = bf16_round(x.astype(np.float32))
    return cfg, kind_m[1], wd, folder, x, T


def test_a_far_key_decides_the_output_just_inside_the_window_and_not_just_outside(tmp_path):
    from purhie_b200.parts import PartProbe
    window, at = 180, 37
    for dtype in ("float32", "bfloat16"):
        cfg, m, w, folder, x, T = far_key_case("F32" if dtype == "float32" else "BF16", tmp_path / dtype, window, at)
        ref = P.latent_attention_mixer(x.astype(np.float64), w, "l0.mix.", m, cfg["norm"]["eps"])
        edge = at + window                                                            # the first row that no longer sees `at`
        assert np.abs(ref[edge] - ref[edge - 1]).max() > 0.2 * np.abs(ref).max()       # the plain implementation shows the step
        p = PartProbe("mixer", *part_of(cfg, 0, "mixer"), dtype=dtype)
        p.bind_folder(folder)
        p.mixer_cache(8, 64, 2)
        tol = 2e-4 if dtype == "float32" else 4e-2
        close(mixer_in_pieces(p, x, [T], 1), ref, tol)
        close(mixer_in_pieces(p, x, [edge - 3] + [1] * (T - edge + 3), 2), ref, tol)   # the edge passes while decoding
        close(mixer_in_pieces(p, x, [edge - 1, 2, T - edge - 1], 1), ref, tol)         # and inside a two-token portion


def test_lightning_mixer_alone_cut_batched_and_in_a_slot_used_again(models):
    from purhie_b200.parts import PartProbe
    for name, layer, dtype in (("A", 1, "float32"), ("A", 2, "float32"), ("B", 0, "float32"), ("C", 1, "bfloat16"), ("C", 1, "float32")):
        folder, cfg, w = models[name, dtype]
        m = cfg["layers"][layer]["mixer"]
        rng = np.random.default_rng(layer)
        xs = {r: rng.normal(0, 1.0, (n, cfg["width"])).astype(np.float32) for r, n in ((1, 150), (2, 7), (3, 1), (4, 40))}
        if dtype == "bfloat16":
            xs = {r: bf16_round(x) for r, x in xs.items()}
        ref = {r: P.lightning_mixer(x.astype(np.float64), w, f"l{layer}.mix.", m, cfg["norm"]["eps"]) for r, x in xs.items()}
        tol = 2e-4 if dtype == "float32" else 3e-2
        p = PartProbe("mixer", *part_of(cfg, layer, "mixer"), dtype=dtype)
        p.bind_folder(folder)
        p.mixer_cache(8, 16, 2)                                  # two state slots
        close(mixer_in_pieces(p, xs[1], [150], 1), ref[1], tol)
        close(mixer_in_pieces(p, xs[1], [1, 2, 70, 2, 64, 11], 1), ref[1], tol)     # the slot again, zeroed; chunk edges inside portions
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


def test_the_first_token_still_shows_hundreds_of_tokens_later_in_a_state_that_never_forgets(tmp_path):
    from purhie_b200.parts import PartProbe
    kind_m = lightning(2, 8, 8, [1.0, 0.5])
    cfg = config(16, 10, [(kind_m, None)])
    w = draw_weights(cfg, 9)
    folder = make_folder(tmp_path, cfg, w)
    x = np.random.default_rng(4).normal(0, 1.0, (400, 16)).astype(np.float32)
    x[1:] *= 0.05                                  # later tokens add little to the state: the first one's part stays visible
    y = x.copy()
    y[0] = np.random.default_rng(5).normal(0, 1.0, 16)
    ref_x = P.lightning_mixer(x.astype(np.float64), f64(w), "l0.mix.", kind_m[1], 1e-5)
    ref_y = P.lightning_mixer(y.astype(np.float64), f64(w), "l0.mix.", kind_m[1], 1e-5)
    assert np.abs(ref_x[-1] - ref_y[-1]).max() > 0.3 * np.abs(ref_x).max()
    p = PartProbe("mixer", *part_of(cfg, 0, "mixer"))
    p.bind_folder(folder)
    p.mixer_cache(8, 8, 2)
    close(mixer_in_pieces(p, y, [1, 200] + [1] * 199, 1), ref_y, 2e-4)
    close(mixer_in_pieces(p, x, [400], 1), ref_x, 2e-4)


def test_routed_feed_forward_alone_with_groups_a_scale_and_a_gated_shared_expert(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("A", 0), ("A", 3), ("B", 0), ("B", 2), ("C", 1), ("A", 1)):
        folder, cfg, w = models[name]
        mlp = cfg["layers"][layer]["mlp"]
        x = np.random.default_rng(layer).normal(0, 1.5, (37, cfg["width"])).astype(np.float32)
        pre = f"l{layer}.mlp."
        ref = P.moe_ff(x.astype(np.float64), w, pre, mlp) if mlp["kind"] == "moe" else P.gated_unit(x.astype(np.float64), w, pre, P.gelu_tanh)
        p = PartProbe("feed_forward", *part_of(cfg, layer, "feed_forward"))
        p.bind_folder(folder)
        close(p.feed_forward(x), ref, 2e-4)
        close(p.feed_forward(x[:1]), ref[:1], 2e-4)                      # one row alone chooses the same experts
    # a group's best expert decides which groups stay: with one of three groups kept, the choice differs from the two best of all
    scores = np.random.default_rng(0).random((200, 6))
    free = np.argsort(-scores, axis=1)[:, :2]
    kept = [P.choose_experts(row, 2, 3, 1) for row in scores]
    assert any(set(a) != set(b) for a, b in zip(free, kept))
    assert all(b[0] // 2 == b[1] // 2 for b in kept)


# ---- tensor-core attention over the latent rows inside whole models ------------------------------------------------
def test_key_splits_of_the_latent_attention_agree_with_the_plain_implementation(tmp_path):
    from purhie_b200.engine import StepEntry
    cfg = config(64, 50, [(LATENTS["c256"][0], dense(64)), (LATENTS["c512"][0], None), (latent(4, 16, 32, 24, 32, 128, None, base=300.0, scale=0.35), None)],
                 loop=(1, 3, 2))
    w = draw_weights(cfg, 8)
    folder = make_folder(tmp_path, cfg, w, "BF16")
    toks = tokens(300, cfg["vocab"], 6)
    ref = P.forward(cfg, f64(w), toks)
    for splits in (1, 3, 0):                                   # whole tiles, three CTAs a tile, the part's own choice
        eng = engine_for(folder, "bfloat16", max_tokens=1024, step_options={"latent_splits": splits})
        close(run_cut(eng, "whole", toks, []), ref, TOL["bfloat16"])
        close(run_cut(eng, "tail", toks, [2, 250] + [1] * 48), ref, TOL["bfloat16"])
        eng.add_request("a"); eng.add_request("b")
        eng.step([StepEntry("a", toks[:200], [])])
        out = eng.step([StepEntry("a", toks[200:201], [0]), StepEntry("b", toks[:130], list(range(130)))])
        close(out[:1], ref[200:201], TOL["bfloat16"])
        close(out[1:], ref[:130], TOL["bfloat16"])
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

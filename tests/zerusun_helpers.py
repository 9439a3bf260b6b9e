"""Small Zerusun configurations and model folders with weights the tests choose themselves."""
import numpy as np

from bozosun_helpers import bf16_round, make_folder, tokens, write_safetensors  # noqa: F401  (re-exported)


def lightning(heads, dim, vdim, decay):
    assert len(decay) == heads
    return ("lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)})


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return ("latent_attention", m)


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups, keep, shared, scale=1.0):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def config(width, vocab, layers, loop=None, eps=1e-5):
    c = {"architecture": "Zerusun", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [{"type": kind, "mixer": m, "mlp": mlp} for (kind, m), mlp in layers]}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# Configurations that differ in every size.  Windows of 1, 3, 8 (a page), 13, 40 and none at all; latents narrower and wider
# than a head; rotated parts of 2, 4, 6 and 12 dimensions, with and without stretched frequencies; one head and five; decays
# from a state that forgets within two tokens to one that never does; values narrower and wider than keys; routers with
# and without real groups, top 1 and top = all kept experts, with and without a shared expert; layers without a
# feed-forward; the repeated stretch at the start, in the middle, at the end, the whole model, once, and not at all.
CONFIG_A = config(48, 80, [
    (latent(3, 8, 4, 12, 10, 20, 13, base=500.0, scaling=(4.0, 64, 16.0, 2.0), scale=0.4), moe(16, 6, 2, 3, 2, 24, scale=1.5)),
    (lightning(2, 8, 16, [0.5, 0.97]), dense(64)),
    (lightning(3, 24, 8, [1.0, 0.8, 0.93]), None),
    (latent(2, 16, 6, 8, 24, 12, 8, scale=0.3), moe(8, 8, 3, 1, 1, 0)),
], loop=(1, 3, 2), eps=1e-6)

CONFIG_B = config(40, 70, [
    (lightning(5, 4, 12, [0.3, 0.6, 0.9, 0.99, 0.999]), moe(24, 4, 1, 4, 2, 16, scale=0.7)),
    (latent(1, 20, 12, 24, 8, 32, 3, base=77.0), dense(56)),
    (latent(5, 4, 2, 4, 16, 6, None, base=1e5, scaling=(16.0, 32, 8.0, 0.5)), moe(12, 9, 6, 3, 2, 40, scale=3.0)),
], loop=(0, 1, 3), eps=1e-3)

# wider layers, stored in bfloat16: a latent of 128 + 32, a state of 64 x 128 per head, the whole model repeated
CONFIG_C = config(128, 200, [
    (latent(4, 32, 32, 64, 64, 128, 40, base=5e5, scaling=(8.0, 128, 32.0, 1.0)), dense(256)),
    (lightning(2, 64, 128, [0.9, 0.995]), moe(64, 8, 2, 4, 2, 128, scale=2.0)),
    (latent(8, 16, 8, 16, 96, 48, 1, base=1e4), moe(32, 4, 2, 2, 1, 64)),
], loop=(0, 3, 2), eps=1e-6)


def draw_weights(cfg, seed, std=0.3):
    """Weights for every tensor the framework says the configuration reads: matrices N(0, 3 std / sqrt(fan_in)) so that
    activations stay of order one, norm weights around 1, biases small but not negligible, the dynamic tanh's alpha in its
    bending range."""
    from purhie_b200.weights import expected_tensors
    rng = np.random.default_rng(seed)
    out = {}
    for name, spec in expected_tensors(cfg).items():
        shape = tuple(spec.shape)
        if name.endswith(".alpha"):
            a = rng.uniform(0.4, 1.1, shape)
        elif name.endswith(".b"):
            a = rng.normal(0.0, 0.2, shape)
        elif name == "loop.step":
            a = rng.normal(0.0, 0.5, shape)
        elif spec.init == "scale":
            a = rng.uniform(0.5, 1.5, shape)
        elif len(shape) == 2:
            a = rng.normal(0.0, std * 3.0 / np.sqrt(shape[1]), shape)
        else:
            a = rng.normal(0.0, std, shape)
        out[name] = bf16_round(np.asarray(a, dtype=np.float32))          # representable in either storage
    return out


def steady_choice(cfg, weights, seed=0):
    """The same weights with a constant input to every router that decides which experts are chosen, a different set in
    every layer: the layer's norm gives 1 in coordinate 0 whatever the token (weight 0, bias 1), and the router's column
    0 lifts the chosen `top`, inside `keep` groups, 40 above all others and within 1 of each other, so that a rounding of
    the router's input cannot change the set while the weights still follow the token."""
    rng = np.random.default_rng(seed)
    out = dict(weights)
    for i, layer in enumerate(cfg["layers"]):
        mlp = layer.get("mlp")
        if not mlp or mlp["kind"] != "moe":
            continue
        r = mlp["router"]
        experts, top = r["experts"], r["top"]
        groups, keep = (r["groups"]["count"], r["groups"]["keep"]) if r.get("groups") else (1, 1)
        per = experts // groups
        kept = rng.permutation(groups)[:keep]
        pool = np.concatenate([np.arange(g * per, (g + 1) * per) for g in kept])
        chosen = rng.permutation(pool)[:top]
        column = np.full(experts, -20.0, dtype=np.float32)
        column[chosen] = 20.0 + rng.uniform(0.0, 1.0, top).astype(np.float32)
        w, b, router = out[f"l{i}.norm1"].copy(), out[f"l{i}.norm1.b"].copy(), out[f"l{i}.mlp.router"].copy()
        w[0], b[0] = 0.0, 1.0
        router[:, 0] = column
        out[f"l{i}.norm1"], out[f"l{i}.norm1.b"], out[f"l{i}.mlp.router"] = w, b, bf16_round(router)
    return out

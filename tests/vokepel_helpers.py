"""Small Vokepel configurations and model folders with weights the tests choose themselves."""
import numpy as np

from bozosun_helpers import bf16_round, make_folder, tokens, write_safetensors  # noqa: F401  (re-exported)


def talking(heads, kv_heads, dim, window, scale=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if softcap is not None:
        m["softcap"] = softcap
    return ("attention", m)


def left_side(heads, kv_heads, dim, vdim, window, rot_dims, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return m


def pair(left, right_width, left_scale=1.0, right_scale=1.0):
    return ("parallel", {"left": left, "right": {"width": right_width}, "left_scale": left_scale, "right_scale": right_scale})


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, loop=None, eps=1e-5, mult=None, logit_scale=None, logit_softcap=None):
    c = {"architecture": "Vokepel", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [{"type": kind, "mixer": m, "mlp": mlp} for (kind, m), mlp in layers]}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    if mult is not None:
        c["residual_mult"] = mult
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    if logit_softcap is not None:
        c["logit_softcap"] = logit_softcap
    return c


# Configurations that differ in every size.  Windows of 1, 3, 8 (a page), 13, 21, 40 and none at all, different from layer
# to layer; groups of 1, 2, 3 and 4 query heads and one kv head for all; heads of 8 to 64; values narrower and wider than
# keys on the left side; rotation over a whole head, part of one, a single pair and none; with and without a cap on the
# scores and on the logits; factors on the residual of 1 (the plain pre-norm path) and others; recurrent widths narrower
# and wider than the model; layers without a feed-forward; the repeated stretch at the start, in the middle, over the
# whole model, once, three times and not at all; a model of one kind of layer only.
CONFIG_A = config(48, 80, [
    (pair(left_side(3, 1, 8, 12, 13, 4, base=500.0, scale=0.4), 40, 0.8, 1.3), dense(64)),
    (talking(4, 2, 12, 21, scale=0.3, softcap=5.0), None),
    (talking(3, 3, 16, 8, scale=0.25), dense(40)),
    (pair(left_side(2, 2, 16, 8, None, 16, base=77.0), 72, 1.5, 0.5), dense(24)),
], loop=(1, 3, 2), eps=1e-6, mult=0.6, logit_scale=1.7, logit_softcap=12.0)

CONFIG_B = config(40, 70, [
    (talking(5, 1, 8, None, scale=0.5, softcap=50.0), dense(56)),
    (pair(left_side(4, 2, 10, 10, 3, 2, base=1e5, scale=0.3), 24, 1.0, 1.0), None),
    (talking(2, 1, 20, 1, scale=0.2, softcap=3.0), dense(16)),
], loop=(0, 1, 3), eps=1e-3)

# wider layers, stored in bfloat16: heads of 64 on the left side, six talking heads of 32, the whole model repeated once
CONFIG_C = config(128, 200, [
    (pair(left_side(4, 1, 64, 32, 40, 32, base=3e5), 160, 0.7, 0.9), dense(256)),
    (talking(6, 2, 32, 40, scale=0.2, softcap=15.0), dense(192)),
    (pair(left_side(2, 1, 32, 64, 70, 0), 96, 1.2, 0.4), None),
], loop=(0, 3, 1), eps=1e-6, mult=0.8, logit_softcap=25.0)


def draw_weights(cfg, seed, std=0.3):
    """Weights for every tensor the framework says the configuration reads: matrices N(0, 3 std / sqrt(fan_in)) so that
    activations stay of order one, norm weights around 1, biases small but not negligible, the heads' mixing matrix near
    the identity, distance slopes of either sign with positive rates, sinks of the size of a score."""
    from purhie_b200.weights import expected_tensors
    rng = np.random.default_rng(seed)
    out = {}
    for name, spec in expected_tensors(cfg).items():
        shape = tuple(spec.shape)
        if name.endswith(".talk"):
            a = np.eye(shape[0]) + rng.normal(0.0, 0.3, shape)
        elif name.endswith(".r1"):
            a = rng.normal(0.0, 0.4, shape)
        elif name.endswith(".r2"):
            a = rng.uniform(0.05, 2.0, shape)
        elif name.endswith(".sink"):
            a = rng.normal(0.0, 1.5, shape)
        elif name.endswith(".b"):
            a = rng.normal(0.0, 0.5, shape)
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

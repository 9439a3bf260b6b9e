"""A plain, slow Zerusun forward pass: one whole sequence from position 0, no cache, one function per mechanism.

It shares no code with ``purhie_b200``: it reads ``config.json`` with ``json`` and the weight file by its byte
layout, and states every equation directly.  Everything runs in float64.

The design in short (names of config.json in quotes):

* e = DyT(embed[token]; "embed.norm"), DyT(a; n) = tanh(alpha_n a) * w_n + b_n (no statistics of the row at all).
* Layers run in the order of "layers", except that the layers "loop.start" .. "loop.stop" - 1 run "loop.times" times
  in a row before the rest follows.  At the start of pass t the stream is re-made from itself and from e:
  x <- W_in [x ; e] + step[t]  (``loop.in`` [width, 2 width], ``loop.step`` [times, width]).
* A layer: h = DyT(x; norm1), x <- x + mixer(h) + ff(h): both parts read the same h.
* Mixer "lightning": q, k, v = silu of their projections; per head S <- d_head S + k v^T, o = S^T q with the constant
  "decay"[head]; the heads' o side by side are RMS-normed as one row, times sigmoid(W_g h), projected.
* Mixer "latent_attention": queries c_q = RMS(W_dq h), q = W_uq c_q, per head "dim" plain and "rot_dim" rotated
  dimensions; W_dkv h gives "kv_rank" values, RMS-normed to the latent c, and "rot_dim" more that are the one rotated
  key part of all heads; per head k = W_uk c and v = W_uv c; scores (q_plain . k_plain + q_rot . k_rot) * "scale" over
  the last "mask.size" positions, softmax, each head's output times sigmoid(W_g h)[head], projected.  Rotation: pairs
  (i, i + dims/2) of the rotated part, frequencies blended between f_i and f_i / factor ("rot.scaling"), cosines and
  sines stretched by 0.1 ln(factor) + 1.
* Feed-forward "dense": W_down (gelu_tanh(W_gate h) * W_up h).  "moe": experts W_down (silu(W_gate h) * W_up h); scores
  softmax(W_router h) over all experts; a group of neighbouring experts counts as its largest score, the best
  "groups.keep" groups stay, the "top" largest scores among them are chosen; weights = chosen scores / (their sum +
  1e-20) * "router.scale"; a shared expert of the same form is added for every token times sigmoid(W_sg h).
* logits = embed DyT(x; "final.norm").
"""
import json
import math
import os
import struct

import numpy as np


# ---- files ---------------------------------------------------------------------------------------------------------
def read_safetensors(path):
    """{name: float64 array (int tables stay int)}: 8-byte little-endian header length, the JSON header (name ->
    dtype, shape, data_offsets), the data."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = data[lo:hi]
        kind = meta["dtype"]
        if kind == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif kind == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif kind == "I32":
            a = np.frombuffer(raw, dtype="<i4").copy()
        else:
            raise ValueError(f"{name}: dtype {kind}")
        out[name] = a.reshape(meta["shape"])
    return out


def read_model(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ---- small functions -----------------------------------------------------------------------------------------------
def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def gelu_tanh(x):
    return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def rms_norm(a, w, eps):
    return a / np.sqrt((a * a).mean(axis=-1, keepdims=True) + eps) * w


def dynamic_tanh(a, w, name):
    return np.tanh(float(w[name + ".alpha"]) * a) * w[name] + w[name + ".b"]


# ---- the decayed state ---------------------------------------------------------------------------------------------
def constant_decay_recurrence(q, k, v, decay):
    """Per head: S_t = decay[head] S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, D]; v [T, H, DV]; decay [H]."""
    T, H, D = q.shape
    o = np.zeros((T, H, v.shape[2]))
    S = np.zeros((H, D, v.shape[2]))
    d = np.asarray(decay, dtype=np.float64)[:, None, None]
    for t in range(T):
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    return o


def lightning_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + "q"].T).reshape(T, H, D)
    k = silu(h @ w[pre + "k"].T).reshape(T, H, D)
    v = silu(h @ w[pre + "v"].T).reshape(T, H, DV)
    o = constant_decay_recurrence(q, k, v, m["decay"]).reshape(T, H * DV)
    o = rms_norm(o, w[pre + "norm"], eps) * sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


# ---- attention through a latent ------------------------------------------------------------------------------------
def rotary_frequencies(rot):
    """Turns per position of pair i, and the stretch of cosines and sines."""
    dims, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, n]: of the first rot.dims dimensions, i turns together with i + dims/2; the rest stay."""
    f, stretch = rotary_frequencies(rot)
    half = rot["dims"] // 2
    out = x.copy()
    for i in range(half):
        angle = positions * f[i]
        c, s = (np.cos(angle) * stretch)[:, None], (np.sin(angle) * stretch)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def window_mask(T, size):
    """visible[i, j]: 0 <= i - j < size (size None: every j <= i)."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) if size else True)


def latent_attention_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, D, R, DV, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T, dtype=np.float64)
    q = (rms_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps) @ w[pre + "uq"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[:, :, :D], rotate(q[:, :, D:], pos, m["rot"])
    down = h @ w[pre + "dkv"].T
    c = rms_norm(down[:, :C], w[pre + "dkv.norm"], eps)
    k_rot = rotate(down[:, None, C:], pos, m["rot"])[:, 0]
    k_plain = (c @ w[pre + "uk"].T).reshape(T, H, D)
    v = (c @ w[pre + "uv"].T).reshape(T, H, DV)
    visible = window_mask(T, (m.get("mask") or {}).get("size"))
    gate = sigmoid(h @ w[pre + "g"].T)
    out = np.zeros((T, H, DV))
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        s = np.where(visible, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[:, a] = (p @ v[:, a]) * gate[:, a:a + 1]
    return out.reshape(T, H * DV) @ w[pre + "o"].T


# ---- feed-forwards -------------------------------------------------------------------------------------------------
def gated_unit(h, w, pre, act):
    return (act(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def choose_experts(scores, top, groups, keep):
    """One token.  The chosen experts in descending order of their scores (the lower index on a tie)."""
    E = len(scores)
    per = E // groups
    best = [scores[g * per:(g + 1) * per].max() for g in range(groups)]
    kept = sorted(range(groups), key=lambda g: (-best[g], g))[:keep]
    allowed = np.full(E, -np.inf)
    for g in kept:
        allowed[g * per:(g + 1) * per] = scores[g * per:(g + 1) * per]
    return sorted(range(E), key=lambda e: (-allowed[e], e))[:top]


def moe_ff(h, w, pre, f):
    r = f["router"]
    z = h @ w[pre + "router"].T
    scores = np.exp(z - z.max(axis=1, keepdims=True))
    scores /= scores.sum(axis=1, keepdims=True)
    g = r.get("groups") or {"count": 1, "keep": 1}
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = choose_experts(scores[t], r["top"], g["count"], g["keep"])
        total = sum(scores[t, e] for e in chosen) + 1e-20
        for e in chosen:
            out[t] += scores[t, e] / total * r.get("scale", 1.0) * gated_unit(h[t:t + 1], w, f"{pre}e{e}.", silu)[0]
    if f.get("shared"):
        out = out + sigmoid(h @ w[pre + "shared.sg"].T) * gated_unit(h, w, pre + "shared.", silu)
    return out


# ---- the model -----------------------------------------------------------------------------------------------------
def run_order(cfg):
    """[(layer, pass or None)]: pass t on the first layer of the t-th time round the loop."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, layer_outputs=None):
    """logits [T, vocab] for one sequence from position 0; layer_outputs (a list) receives x after every layer run."""
    eps = cfg["norm"]["eps"]
    e = dynamic_tanh(w["embed"][np.asarray(tokens)], w, "embed.norm")
    x = e
    for i, t in run_order(cfg):
        layer = cfg["layers"][i]
        pre = f"l{i}."
        if t is not None:
            x = np.concatenate([x, e], axis=1) @ w["loop.in"].T + w["loop.step"][t]
        h = dynamic_tanh(x, w, pre + "norm1")
        if layer["type"] == "lightning":
            y = lightning_mixer(h, w, pre + "mix.", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(h, w, pre + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer {i}: type {layer['type']}")
        f = layer.get("mlp")
        if f is not None:
            y = y + (gated_unit(h, w, pre + "mlp.", gelu_tanh) if f["kind"] == "dense" else moe_ff(h, w, pre + "mlp.", f))
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return dynamic_tanh(x, w, "final.norm") @ w["embed"].T

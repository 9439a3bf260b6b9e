"""A plain, slow Vokepel forward pass: one whole sequence from position 0, no cache, one function per mechanism.

It shares no code with ``purhie_b200``: it reads ``config.json`` with ``json`` and the weight file by its byte
layout, and states every equation directly.  Everything runs in float64.

The design in short (names of config.json in quotes):

* e = embed[token].  Layers run in the order of "layers", except that the layers "loop.start" .. "loop.stop" - 1 run
  "loop.times" times in a row before the rest follows; at the start of pass t the stream is re-made from itself and
  from e: x <- W_in [x ; e] + step[t].
* A layer: x <- x + m rms(mixer)(...) in pre-norm form: x <- x + m * mixer(rms(x; norm1)), then, if the layer has a
  feed-forward, x <- x + m * ff(rms(x; norm2)), m = "residual_mult".
* Mixer "attention": q = W_q h and k = W_k h are RMS-normed over the whole projection (all heads as one row, a weight per
  element); the values are k as projected, before that norm.  A head's score with a key d positions back is
  s = (q . k) * "scale", then softcap * tanh(s / softcap), minus r1_h * ln(1 + r2_h * d); then the heads' scores at one
  (query, key) pair are mixed, s_h <- sum_g talk[h, g] s_g; softmax over the last "mask.size" positions; the heads side
  by side times sigmoid(W_g h); W_o.
* Mixer "parallel": "left_scale" * left(h) + "right_scale" * right(h).  Left: grouped-query attention, interleaved rotary
  pairs (2i, 2i + 1) over the first "rot.dims" dimensions of a head, a sliding window, and a softmax whose denominator
  also holds exp(sink_h).  Right: a minimal gated recurrent unit, z = sigmoid(W_z h + b_z), u = W_x h + b_x, candidate
  c = u + 1/2 where u >= 0 and sigmoid(u) below, S <- (1 - z) S + z c from S = 0, output W_o (S * silu(W_g h)).
* Feed-forward: W_down relu(W_up h)^2.
* logits = cap * tanh(embed rms(x; final.norm) * "logit_scale" / cap), cap = "logit_softcap".
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


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def soft_cap(s, cap):
    return cap * np.tanh(s / cap)


def window_mask(n, size):
    """[n, n] True where query i sees key j: 0 <= i - j < size (size None or 0: every earlier position)."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    d = i - j
    return (d >= 0) & ((d < size) if size else True)


# ---- mechanisms ----------------------------------------------------------------------------------------------------
def rotate_interleaved(x, dims, base):
    """x [n, heads, dim] at positions 0 .. n-1: pairs (2i, 2i+1) of the first `dims` dimensions turned by p * base^(-2i/dims)."""
    n = x.shape[0]
    out = x.copy()
    if not dims:
        return out
    f = base ** (-2.0 * np.arange(dims // 2) / dims)
    a = np.arange(n)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def distance_bias(n, r1, r2):
    """[heads, n, n]: r1_h * ln(1 + r2_h * (i - j)) for j <= i (0 elsewhere)."""
    d = np.maximum(np.arange(n)[:, None] - np.arange(n)[None, :], 0).astype(np.float64)
    return r1[:, None, None] * np.log1p(r2[:, None, None] * d[None])


def talking_attention(h, w, p, m, eps):
    """Mixer "attention": keys double as values, norms over the whole projection, capped and distance-biased scores that
    are mixed across heads before the softmax, a sigmoid gate on the heads' outputs."""
    n = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = h @ w[p + "q"].T
    k = h @ w[p + "k"].T
    v = k.reshape(n, G, D)                                         # the values: k as projected
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(n, H, D)
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(n, G, D)
    rep = H // G
    s = np.einsum("ihd,jhd->hij", q, np.repeat(k, rep, axis=1)) * m["scale"]
    if m.get("softcap"):
        s = soft_cap(s, m["softcap"])
    s = s - distance_bias(n, w[p + "r1"], w[p + "r2"])
    s = np.einsum("hg,gij->hij", w[p + "talk"], s)
    seen = window_mask(n, m.get("mask", {}).get("size") if m.get("mask") else None)
    s = np.where(seen[None], s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    pr = e / e.sum(axis=-1, keepdims=True)
    o = np.einsum("hij,jhd->ihd", pr, np.repeat(v, rep, axis=1)).reshape(n, H * D)
    o = o * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def sink_attention(h, w, p, m):
    """The left mixer: grouped-query attention with interleaved rotary pairs, a sliding window and a sink in the softmax."""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(n, H, D)
    k = (h @ w[p + "k"].T).reshape(n, G, D)
    v = (h @ w[p + "v"].T).reshape(n, G, V)
    rot = m.get("rot")
    if rot:
        q = rotate_interleaved(q, rot["dims"], rot["base"])
        k = rotate_interleaved(k, rot["dims"], rot["base"])
    rep = H // G
    s = np.einsum("ihd,jhd->hij", q, np.repeat(k, rep, axis=1)) * m["scale"]
    seen = window_mask(n, m.get("mask", {}).get("size") if m.get("mask") else None)
    s = np.where(seen[None], s, -np.inf)
    sink = w[p + "sink"][:, None, None]
    top = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - top)
    pr = e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - top))
    o = np.einsum("hij,jhd->ihd", pr, np.repeat(v, rep, axis=1)).reshape(n, H * V)
    return o @ w[p + "o"].T


def min_gru_candidate(u):
    return np.where(u >= 0, u + 0.5, sigmoid(u))


def min_gru(h, w, p, state=None):
    """The right mixer: S_t = (1 - z_t) S_(t-1) + z_t c_t element by element, from S = 0 (or `state`)."""
    z = sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    c = min_gru_candidate(h @ w[p + "x"].T + w[p + "x.b"])
    s = np.zeros(z.shape[1]) if state is None else state.copy()
    states = np.empty_like(z)
    for t in range(z.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * c[t]
        states[t] = s
    return (states * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def side_by_side(h, w, p, m):
    return m["left_scale"] * sink_attention(h, w, p + "left.", m["left"]) + m["right_scale"] * min_gru(h, w, p + "right.")


def squared_relu_unit(h, w, p):
    return (np.maximum(h @ w[p + "up"].T, 0.0) ** 2) @ w[p + "down"].T


def layer(x, i, cfg, w):
    l = cfg["layers"][i]
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    p = f"l{i}."
    h = rms_norm(x, w[p + "norm1"], eps)
    if l["type"] == "attention":
        x = x + mult * talking_attention(h, w, p + "mix.", l["mixer"], eps)
    elif l["type"] == "parallel":
        x = x + mult * side_by_side(h, w, p + "mix.", l["mixer"])
    else:
        raise ValueError(l["type"])
    if l.get("mlp"):
        x = x + mult * squared_relu_unit(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
    return x


def run_order(cfg):
    """[(layer, pass, first of its pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, 0, False) for i in range(n)]
    order = [(i, 0, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, 0, False) for i in range(loop["stop"], n)]


def head(x, cfg, w):
    y = rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return soft_cap(y, cap) if cap else y


def forward(cfg, w, tokens, layers_out=None):
    """Logits [n, vocab] of one whole sequence; `layers_out`, a list, receives the stream after every layer run."""
    e = w["embed"][np.asarray(tokens)]
    x = e
    for i, t, first in run_order(cfg):
        if first:
            x = np.concatenate([x, e], axis=-1) @ w["loop.in"].T + w["loop.step"][t]
        x = layer(x, i, cfg, w)
        if layers_out is not None:
            layers_out.append(x.copy())
    return head(x, cfg, w)

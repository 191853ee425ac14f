"""A plain, slow Nomutar: every mechanism as one numpy function over a whole sequence, float64 throughout.

Nothing here is shared with the package: no cache, no state carried between calls, no kernels.  A sequence goes in
whole and every position's result comes out, so that the engine's cuttings (portions, decoding, batches) can be held
against it.  Weights are a dict of numpy arrays by tensor name; the configuration is the plain dict of config.json.

Notation: T tokens, E the model's width, H query heads, G key/value heads, D key width per head, V value width per head.
"""
import math

import numpy as np

F = np.float64


# ---- small functions --------------------------------------------------------------------------------------------------
def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def soft_cap(z, cap):
    """cap * tanh(z / cap)."""
    return cap * np.tanh(z / cap)


def grouped_rms_norm(x, w, eps, groups):
    """The last axis in `groups` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps); then times w."""
    x = x.astype(F)
    shape = x.shape
    parts = x.reshape(shape[:-1] + (groups, shape[-1] // groups))
    parts = parts / np.sqrt((parts * parts).mean(axis=-1, keepdims=True) + eps)
    return parts.reshape(shape) * w.astype(F)


def causal_filter(u, taps_w):
    """y[t, c] = sum_j w[c, j] u[t - taps + 1 + j, c], u = 0 before the sequence.  u [T, channels]; w [channels, taps]."""
    T, n = u.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, n), dtype=F), u.astype(F)], axis=0)
    y = np.zeros((T, n), dtype=F)
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j].astype(F)[None, :]
    return y


# ---- embedding --------------------------------------------------------------------------------------------------------
def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """The row of the pair table for every position: the hash of (token before, token), or row `buckets` at position 0."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return np.asarray(rows, dtype=np.int64)


def embed(tokens, table, scale, pair_table=None, buckets=0, mul_prev=0, mul_cur=0):
    x = table[np.asarray(tokens)].astype(F) * scale
    if pair_table is not None:
        x = x + pair_table[pair_rows(tokens, buckets, mul_prev, mul_cur)].astype(F)
    return x


# ---- rotations --------------------------------------------------------------------------------------------------------
def plain_frequencies(base, dims):
    i = np.arange(dims // 2, dtype=F)
    return np.power(F(base), -2.0 * i / dims)


def banded_frequencies(base, dims, factor, low, high, original):
    """Short wavelengths keep their frequency, long ones are divided by `factor`, those between are blended by how many
    turns they make in `original` positions."""
    f = plain_frequencies(base, dims)
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out[i] = fi
        elif wavelength > original / low:
            out[i] = fi / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def ramped_frequencies(base, dims, factor, original, fast, slow):
    """Frequencies blended between f_i and f_i / factor by a ramp over the pair index, and the factor on cosines and sines."""
    f = plain_frequencies(base, dims)

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    i = np.arange(dims // 2, dtype=F)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freq, layout, magnitude=1.0, sign=1.0):
    """The first 2 len(freq) entries of the last axis in pairs turned by sign * position * freq[i]: pair i is
    (i, i + len(freq)) in the "halves" layout and (2i, 2i + 1) in the "neighbours" layout.  x [T, heads, n]."""
    out = x.astype(F).copy()
    n = len(freq)
    if n == 0:
        return out
    angle = sign * np.asarray(positions, dtype=F)[:, None] * np.asarray(freq, dtype=F)[None, :]
    c, s = (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]
    if layout == "halves":
        a, b = out[..., :n].copy(), out[..., n:2 * n].copy()
        out[..., :n] = a * c - b * s
        out[..., n:2 * n] = b * c + a * s
    else:
        a, b = out[..., 0:2 * n:2].copy(), out[..., 1:2 * n:2].copy()
        out[..., 0:2 * n:2] = a * c - b * s
        out[..., 1:2 * n:2] = b * c + a * s
    return out


# ---- attention --------------------------------------------------------------------------------------------------------
def masked_softmax_attention(q, k, v, scale, window=None, cap=None, sink=None):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V].  Position i sees j <= i (and i - j < window).  `cap`: scores
    go through cap * tanh(score / cap).  `sink` [H]: exp(sink_h) joins the denominator of head h (no key, no value)."""
    T, H, D = q.shape
    G, V = k.shape[1], v.shape[2]
    out = np.zeros((T, H, V), dtype=F)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g].astype(F) @ q[i, h].astype(F)) * scale
            if cap is not None:
                s = soft_cap(s, cap)
            m = s.max() if sink is None else max(s.max(), float(sink[h]))
            e = np.exp(s - m)
            denom = e.sum() + (0.0 if sink is None else math.exp(float(sink[h]) - m))
            out[i, h] = (e / denom) @ v[lo:i + 1, g].astype(F)
    return out


def attention_mixer(h, w, prefix, m, kind, eps):
    """One of the three attention mixers on its input h [T, E]; `m`: the mixer's entry of the configuration."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = h @ w[prefix + "q"].astype(F).T
    k = h @ w[prefix + "k"].astype(F).T
    v = h @ w[prefix + "v"].astype(F).T
    if kind == "attention_2":
        q, k, v = q + w[prefix + "q.b"].astype(F), k + w[prefix + "k.b"].astype(F), v + w[prefix + "v.b"].astype(F)
    else:
        q = grouped_rms_norm(q, w[prefix + "q.norm"], eps, 1)
        k = grouped_rms_norm(k, w[prefix + "k.norm"], eps, 1)
    q, k, v = q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, V)
    rot = m.get("rot") or {}
    dims, base, sc = rot.get("dims", 0), rot.get("base", 10000.0), rot.get("scaling")
    layout = "neighbours" if kind == "attention_2" else "halves"
    mag = 1.0
    if dims:
        if sc is None:
            freq = plain_frequencies(base, dims)
        elif kind == "attention_2":
            freq, mag = ramped_frequencies(base, dims, sc["factor"], sc["original"], sc["fast"], sc["slow"])
        else:
            freq = banded_frequencies(base, dims, sc["factor"], sc["low"], sc["high"], sc["original"])
        q, k = rotate(q, pos, freq, layout, mag), rotate(k, pos, freq, layout, mag)
    window = (m.get("mask") or {}).get("size")
    if kind == "attention":
        vfreq = plain_frequencies(base, V)
        v = rotate(v, pos, vfreq, layout)
        o = masked_softmax_attention(q, k, v, m["scale"], window, m.get("softcap"), w[prefix + "sink"].astype(F))
        o = rotate(o, pos, vfreq, layout, sign=-1.0)
    elif kind == "attention_2":
        o = masked_softmax_attention(q, k, v, m["scale"], window, m.get("softcap"), np.zeros(H))
    else:
        o = masked_softmax_attention(q, k, v, m["scale"])
    return o.reshape(T, H * V) @ w[prefix + "o"].astype(F).T


# ---- feed-forward -----------------------------------------------------------------------------------------------------
def gated_unit(h, gate, up, down):
    return (silu(h @ gate.astype(F).T) * (h @ up.astype(F).T)) @ down.astype(F).T


def routed_experts(h, w, prefix, experts, top, margins=None):
    """Each row's `top` experts by the largest router logits, weighted by the softmax over those logits alone.
    `margins`, a list, receives per row how far the last chosen logit lies above the first one left out, as a fraction
    of the spread (standard deviation) of the row's logits."""
    z = h @ w[prefix + "router"].astype(F).T + w[prefix + "router.b"].astype(F)
    out = np.zeros_like(h)
    if margins is not None:
        ranked = -np.sort(-z, axis=1)
        margins.append((ranked[:, top - 1] - ranked[:, top]) / (z.std(axis=1) + 1e-30) if top < experts else np.full(h.shape[0], np.inf))
    for t in range(h.shape[0]):
        chosen = np.argsort(-z[t], kind="stable")[:top]
        p = np.exp(z[t, chosen] - z[t, chosen].max())
        p /= p.sum()
        for e, pe in zip(chosen, p):
            out[t] += pe * gated_unit(h[t:t + 1], w[f"{prefix}e{e}.gate"], w[f"{prefix}e{e}.up"], w[f"{prefix}e{e}.down"])[0]
    return out


def feed_forward(h, w, prefix, mlp, margins=None):
    if mlp["kind"] == "dense":
        return gated_unit(h, w[prefix + "gate"], w[prefix + "up"], w[prefix + "down"])
    out = routed_experts(h, w, prefix, mlp["router"]["experts"], mlp["router"]["top"], margins)
    if mlp.get("shared") is not None:
        s = prefix + "shared."
        out = out + gated_unit(h, w[s + "gate"], w[s + "up"], w[s + "down"]) * sigmoid(h @ w[s + "sg"].astype(F).T)
    return out


# ---- the model --------------------------------------------------------------------------------------------------------
def layer_order(cfg):
    n, loop = len(cfg["layers"]), cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = list(range(loop["start"]))
    for _ in range(loop["times"] if loop["stop"] > loop["start"] else 0):
        order += list(range(loop["start"], loop["stop"]))
    return order + list(range(loop["stop"], n))


def forward(cfg, w, tokens, streams=None, margins=None):
    """Logits [T, vocab] of a whole sequence; `streams`, a list, receives the residual stream after every layer run;
    `margins`, a list, one array [T] per routed feed-forward run: the margin of each row's choice of experts."""
    eps, groups, mult = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg.get("residual_mult", 1.0)
    emb = cfg.get("embedding") or {}
    bi = emb.get("bigram")
    taps = (cfg.get("canon") or {}).get("taps", 0)
    x = embed(tokens, w["embed"], emb.get("scale", 1.0), w["bigram"] if bi else None,
              *((bi["buckets"], bi["mul_prev"], bi["mul_cur"]) if bi else ()))
    for i in layer_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        h = grouped_rms_norm(x, w[p + "norm1"], eps, groups)
        hm = h + causal_filter(h, w[p + "canon1"]) if taps else h
        y = attention_mixer(hm, w, p + "mix.", layer["mixer"], layer["type"], eps)
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, w, p + "mlp.", layer["mlp"], margins)
        x = x + mult * y
        if streams is not None:
            streams.append(x.copy())
    logits = grouped_rms_norm(x, w["final.norm"], eps, groups) @ w["head"].astype(F).T
    cap = cfg.get("logit_softcap")
    return soft_cap(logits, cap) if cap else logits
